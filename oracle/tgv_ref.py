"""CPU restatement of the reference's unrolled FISTA TGV-inpainting layer (cudaTGV/cudaCode/TGVInpaintFistaBetas.cu).
TEST INFRASTRUCTURE ONLY.

State per channel: a primary plane u and two auxiliary planes v1, v2 (second-order TGV).  Tensors (torch, CPU):
  b [N,C,H,W]; c [N,1,H,W]; dx = [wx, beta_x] and dy = [wy, beta_y] as [N,2,H,W];
  init / solution / upstream gradient / init gradient: [N,3,C,H,W] (u, v1, v2) -- the same memory as [N,3C,H,W].
The reference handles N == 1; a batch is N independent problems (each with its own Lipschitz constant).

Formulation.  The reference gathers three triangles per pixel; here every triangle anchored at p is evaluated once
(weights already multiplied by L, differences across the image border are 0):
  z1 = u[p+x]-u[p]-v1[p],  z2 = u[p+y]-u[p]-v2[p],  Hu = min(1, delta*rsqrt(wy z2^2 + wx z1^2))
  Fx = wx z1 Hu,  Fy = wy z2 Hu
  for j in 1,2:  a1 = vj[p+x]-vj[p], a2 = vj[p+y]-vj[p], Hj = min(1, delta*rsqrt(beta_j (a1^2+a2^2))),
                 Gjx = beta_j a1 Hj, Gjy = beta_j a2 Hj
  u_half = u + Fx + Fy - Fx[p-x] - Fy[p-y]
  v1'    = v1 + G1x + G1y - G1x[p-x] - G1y[p-y] + Fx        v2' likewise with Fy
(kernel :1546-1776).  The reverse sweep is the adjoint of this in the same divergence shape (:224-644, :1061-1473).

Pinned by golden vectors from the reference's own kernels (tests/golden/tgv_reference_cuda.npz) and, in exact mode,
by torch.autograd."""
from __future__ import annotations

import math
from typing import List, Optional

import numpy as np
import torch

from oracle.tv_ref import (IdState, checkpoint_schedule, effective_iterations, step_sizes, prox_huber, _prox_reverse,
                           rederive_y)

DELTA_U = float(np.float32(0.2))          # __HDelta2__    :58
DELTA_V1 = float(np.float32(0.2))         # __HDeltaY1__   :59
DELTA_V2 = float(np.float32(0.2))         # __HDeltaY2__   :60
CLIP_LOCAL_GRAD = 2000.0                  # clipLocalGrad  :78
LOCAL_GX_MULT = float(np.float32(0.1))    # localGXMult    :89
GLOBAL_G_MULT = float(np.float32(0.1))    # globalGMult    :93
KILL_T = 35.0                             # TGVInpaintFistaHelp.cu:29
SCALE_T = 10.0
MEMORY_T = 0.95
MAX_TOLERANCE = 5000000.0                 # _maxTolerance_ Help.cu:41
LIP_FLOOR = float(np.float32(32.000001))  # max(12, 8*beta) + 1e-6 stored in a float (:2516)


def _sx(a):      # a[p-x], zero at w == 0
    z = torch.zeros_like(a)
    z[..., :, 1:] = a[..., :, :-1]
    return z


def _sy(a):      # a[p-y], zero at h == 0
    z = torch.zeros_like(a)
    z[..., 1:, :] = a[..., :-1, :]
    return z


def _px(a):      # a[p+x], zero at w == W-1
    z = torch.zeros_like(a)
    z[..., :, :-1] = a[..., :, 1:]
    return z


def _py(a):      # a[p+y], zero at h == H-1
    z = torch.zeros_like(a)
    z[..., :-1, :] = a[..., 1:, :]
    return z


def lipschitz_inverse(dx: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """Per image 1/(max(32.000001, max_p lip(p)) + 0.01) in fp32 (:101-148, :2513-2527).  Returns [N,1,1,1] float32.

    The kernel's beta reads at (w, h-1) under a w > 0 guard and at (w-1, h) under an h > 0 guard rely on clamp-to-edge
    texture addressing; both are reproduced."""
    wx, bx = dx[:, 0:1].float(), dx[:, 1:2].float()
    wy, by = dy[:, 0:1].float(), dy[:, 1:2].float()
    n, _, H, W = wx.shape
    hh = torch.arange(H).view(1, 1, H, 1)
    ww = torch.arange(W).view(1, 1, 1, W)
    z = torch.zeros_like(wx)
    wx_0 = torch.where(ww > 0, _sx(wx), z)
    wx_1 = torch.where(ww < W - 1, wx, z)
    wy_0 = torch.where(hh > 0, _sy(wy), z)
    wy_1 = torch.where(hh < H - 1, wy, z)

    def clamp_up(a):      # a[max(h-1,0)][w]
        return a[..., torch.clamp(torch.arange(H) - 1, min=0), :]

    def clamp_left(a):    # a[h][max(w-1,0)]
        return a[..., :, torch.clamp(torch.arange(W) - 1, min=0)]

    def aux(beta, w_own):
        b_1y = torch.where(hh < H - 1, beta, z)
        b_1x = torch.where(ww < W - 1, beta, z)
        b_0x = torch.where(ww > 0, clamp_up(beta), z)          # (w + 0.5, h - 0.5) guarded by w > 0
        b_0y = torch.where(hh > 0, clamp_left(beta), z)        # (w - 0.5, h + 0.5) guarded by h > 0
        out = torch.where(hh > 0, 2 * b_0y, z) + torch.where(ww > 0, 2 * b_0x, z)
        return out + 2 * b_1x + 2 * b_1y + 3 * w_own

    weightx = torch.where(hh > 0, 3 * wy_0, z) + torch.where(ww > 0, 3 * wx_0, z) + 3 * (wy_1 + wx_1)
    lip = torch.maximum(weightx, torch.maximum(aux(bx, wx_1), aux(by, wy_1)))
    mx = torch.clamp(lip.amax(dim=(1, 2, 3), keepdim=True), min=LIP_FLOOR).float()
    denom = (mx + torch.tensor(0.01, dtype=torch.float32)).float()          # float + float
    return (1.0 / denom.double()).float()                                    # 1. / float -> double -> float


class _W:
    """Scaled, masked weights of one problem batch."""

    def __init__(self, dx, dy, dtype, L=None):
        self.L32 = lipschitz_inverse(dx, dy) if L is None else L
        L = self.L32.to(dtype)
        H, W = dx.shape[-2:]
        self.mx = torch.ones(1, 1, H, W, dtype=dtype)
        self.mx[..., :, -1] = 0
        self.my = torch.ones(1, 1, H, W, dtype=dtype)
        self.my[..., -1, :] = 0
        # thrust::transform(L * _1) on float data: double product rounded to float (:2529-2533); inputs untouched
        sc = (lambda a: (a.double() * self.L32.double()).float().to(dtype)) if dtype == torch.float32 else (lambda a: a.to(dtype) * L)
        self.wx = sc(dx[:, 0:1]) * self.mx
        self.wy = sc(dy[:, 0:1]) * self.my
        self.bx = sc(dx[:, 1:2])
        self.by = sc(dy[:, 1:2])


def _rsqrt(a):
    return torch.where(a > 0, 1.0 / torch.sqrt(torch.where(a > 0, a, torch.ones_like(a))), torch.full_like(a, float("inf")))


def _triangles(u, v1, v2, Wt: _W):
    """All per-triangle quantities of one iterate.  u, v1, v2: [N,C,H,W]."""
    z1 = Wt.mx * (_px(u) - u - v1)
    z2 = Wt.my * (_py(u) - u - v2)
    r_u = _rsqrt(Wt.wy * z2 * z2 + Wt.wx * z1 * z1)
    Hu = torch.clamp(r_u * DELTA_U, max=1.0)
    out = {"z1": z1, "z2": z2, "r_u": r_u, "Hu": Hu}
    for j, (v, beta, d) in enumerate(((v1, Wt.bx, DELTA_V1), (v2, Wt.by, DELTA_V2)), start=1):
        a1 = Wt.mx * (_px(v) - v)
        a2 = Wt.my * (_py(v) - v)
        r = _rsqrt(beta * (a1 * a1 + a2 * a2))
        out[f"a1_{j}"], out[f"a2_{j}"], out[f"r_{j}"], out[f"H_{j}"] = a1, a2, r, torch.clamp(r * d, max=1.0)
    return out


def forward_iteration(y, x_prev, b, c, Wt: _W, t: float):
    """One forward launch (:1546-1776).  y, x_prev: [N,3,C,H,W].  Returns (y_next, x_next, x_half) where x_half holds
    the pre-prox u and the new v1, v2 -- exactly what the *_writexk05 kernels store (:2146-2196)."""
    u, v1, v2 = y[:, 0], y[:, 1], y[:, 2]
    T = _triangles(u, v1, v2, Wt)
    Fx = Wt.wx * T["z1"] * T["Hu"]
    Fy = Wt.wy * T["z2"] * T["Hu"]
    u_half = u + Fx + Fy - _sx(Fx) - _sy(Fy)
    news = []
    for j, (v, beta, F) in enumerate(((v1, Wt.bx, Fx), (v2, Wt.by, Fy)), start=1):
        Gx = beta * T[f"a1_{j}"] * T[f"H_{j}"]
        Gy = beta * T[f"a2_{j}"] * T[f"H_{j}"]
        news.append(v + Gx + Gy - _sx(Gx) - _sy(Gy) + F)
    x_u = prox_huber(u_half, b, c)
    x_next = torch.stack([x_u, news[0], news[1]], dim=1)
    y_next = x_next + t * (x_next - x_prev)
    x_half = torch.stack([u_half, news[0], news[1]], dim=1)
    return y_next, x_next, x_half


def tgv_forward_history(dx, dy, c, b, init, its: int, dtype=torch.float64):
    """Host loop of FistaTGVHuberB2_id::forward (:2475-2618).  init: [N,3,C,H,W].
    Returns (solution, hist [its_eff,N,3,C,H,W], ckpt_y [K,N,3,C,H,W], ckpt_x [K,...], L [N,1,1,1])."""
    Wt = _W(dx, dy, dtype)
    Wt5 = _expand(Wt)
    b = b.to(dtype)
    c = c.to(dtype)
    x = init.to(dtype).clone()
    y = init.to(dtype).clone()
    sched = checkpoint_schedule(its)
    steps = step_sizes(its)
    hist, cky, ckx = [], [], []
    for g in range(effective_iterations(its)):
        if g in sched:
            cky.append(y.clone())
            ckx.append(x.clone())
        y, x, xh = forward_iteration(y, x, b, c, Wt5, steps[g])
        hist.append(xh)
    return x, torch.stack(hist), torch.stack(cky), torch.stack(ckx), Wt.L32


def _expand(Wt: _W) -> _W:
    """Weights are [N,1,H,W]; the state planes are [N,C,H,W]: broadcasting over C works as is."""
    return Wt


# ---------------------------------------------------------------------------------------------------------------
# reverse sweep
# ---------------------------------------------------------------------------------------------------------------
def laplacian_transpose(y, g, Wt: _W, typo: bool):
    """Adjoint of the gradient step at y applied to g (both [N,3,C,H,W]) plus the weight gradients (:303-503).

    typo=True reproduces the reference's non-segment-start kernels, where the Huber-derivative factor of the v2 term
    that arrives from the triangle above is W / rsqrt(A)^2 instead of W * rsqrt(A)^2 (:355, :804); the segment-start
    kernel (:1061-1473) has the consistent form.
    Returns (ybar [N,3,C,H,W], gwx, gbx, gwy, gby each [N,1,H,W], locally scaled by localGXMult)."""
    u, v1, v2 = y[:, 0], y[:, 1], y[:, 2]
    gu, g1, g2 = g[:, 0], g[:, 1], g[:, 2]
    T = _triangles(u, v1, v2, Wt)
    Hu, r_u = T["Hu"], T["r_u"]
    act = Hu < 1.0
    zero = torch.zeros_like(Hu)
    dW = torch.where(act, Hu * torch.where(act, r_u, zero) ** 2, zero)
    Ex = gu - _px(gu) + g1                     # dyij_1 (:436)
    Ey = gu - _py(gu) + g2
    a1 = T["z1"] * Wt.wx
    a2 = T["z2"] * Wt.wy
    S = a1 * Ex + a2 * Ey
    psi1 = Wt.wx * Hu * Ex - dW * a1 * S
    psi2 = Wt.wy * Hu * Ey - dW * a2 * S
    ubar = gu - psi1 - psi2 + _sx(psi1) + _sy(psi2)
    gwx = LOCAL_GX_MULT * (Ex * T["z1"] * Hu - 0.5 * T["z1"] * T["z1"] * dW * S)         # :446, :459
    gwy = LOCAL_GX_MULT * (Ey * T["z2"] * Hu - 0.5 * T["z2"] * T["z2"] * dW * S)
    outs = [ubar]
    gbs = []
    for j, (gj, beta, psi) in enumerate(((g1, Wt.bx, psi1), (g2, Wt.by, psi2)), start=1):
        b1, b2, H, r = T[f"a1_{j}"], T[f"a2_{j}"], T[f"H_{j}"], T[f"r_{j}"]
        actj = H < 1.0
        rr = torch.where(actj, r, zero)
        dWj = torch.where(actj, H * rr * rr, zero)
        E1 = Wt.mx * (gj - _px(gj))
        E2 = Wt.my * (gj - _py(gj))
        Sj = b1 * E1 + b2 * E2
        chi_x = beta * (H * E1 - dWj * beta * b1 * Sj)
        chi_y = beta * (H * E2 - dWj * beta * b2 * Sj)
        chi_y_down = chi_y
        if typo and j == 2:
            A = beta * (b1 * b1 + b2 * b2)
            dW_typo = torch.where(actj, H * A, zero)                 # W / hub^2 with hub = rsqrt(A)   (:355)
            chi_y_down = beta * (H * E2 - dW_typo * beta * b2 * Sj)
        outs.append(gj - psi - chi_x - chi_y + _sx(chi_x) + _sy(chi_y_down))
        gbs.append(LOCAL_GX_MULT * (Sj * H - 0.5 * (b1 * b1 + b2 * b2) * dWj * beta * Sj))       # :467, :477
    s = lambda a: a.sum(dim=1, keepdim=True)
    return torch.stack(outs, dim=1), s(gwx), s(gbs[0]), s(gwy), s(gbs[1])


def reverse_iteration(y, g_in, acc, x_half_u, b, c, Wt: _W, t: float, typo: bool):
    """One reverse launch (:224-644).  Returns (g_out, xbar, acc_next, dgc, dgb, gwx, gbx, gwy, gby)."""
    ybar, gwx, gbx, gwy, gby = laplacian_transpose(y, g_in, Wt, typo)
    xbar = torch.clamp(acc + (1.0 + t) * ybar, -CLIP_LOCAL_GRAD, CLIP_LOCAL_GRAD)        # :577-602
    acc_next = -t * ybar
    g_u, dgc, dgb = _prox_reverse(xbar[:, 0], x_half_u, b, c)
    g_out = torch.stack([g_u, xbar[:, 1], xbar[:, 2]], dim=1)
    return g_out, xbar, acc_next, dgc, dgb, gwx, gbx, gwy, gby


def check_grad_update(g: torch.Tensor, av_current: float):
    """NaN/Inf -> 0, |g| clamped to 5e6, running mean of |g| (TGVInpaintFistaHelp.cu:151-176)."""
    flat = g.reshape(-1).clone()
    if bool(torch.isfinite(flat).all()):
        flat = torch.clamp(flat, -MAX_TOLERANCE, MAX_TOLERANCE)
        av = float(flat.abs().double().mean()) if flat.numel() else 0.0
        return flat.reshape(g.shape), av
    av = 0.0
    vals = flat.tolist()
    for i, v in enumerate(vals):
        if math.isfinite(v):
            tca = min(abs(v), MAX_TOLERANCE)
            vals[i] = math.copysign(tca, v)
            step = i / (i + 1.0)
            av = (1.0 - step) * tca + step * av
        else:
            vals[i] = 0.0
            av = av_current * 1000.0
    return torch.tensor(vals, dtype=g.dtype).reshape(g.shape), av


def update_correct_av_step(run, av_gc, av_state, g, run_step_in):
    """TGVInpaintFistaHelp.cu:119-148."""
    run_step = min(MEMORY_T, run_step_in)
    if run >= 10 and av_state * KILL_T < av_gc:
        return torch.zeros_like(g), av_state * run_step + (1.0 - run_step) * SCALE_T * av_state
    if run >= 10 and av_state * SCALE_T < av_gc:
        mult = SCALE_T * av_state / av_gc
        return g * mult, av_state * run_step + (1.0 - run_step) * av_gc * mult
    return g, av_state * run_step + (1.0 - run_step) * av_gc


def tgv_backward(dx, dy, c, b, grad_out, its: int, hist, ckpt_y, dtype=torch.float64, exact: bool = False,
                 state: Optional[IdState] = None, ys_exact=None):
    """Host loop of FistaTGVHuberB2_id::backward (:2621-3063) on a given history (x_half per iteration) and the
    checkpointed y.

    exact=False reproduces the reference: y for the Jacobian is rebuilt (u) / taken from the stored new iterate
    (v1, v2) (:1478-1541), the checkpointed y_g is used at segment starts, the v2 factor typo is active away from
    segment starts, the init gradient is dL/dx_1.  exact=True uses the true y_{g+1} (ys_exact[g+1]), no typo, and
    back-propagates the first step to init; L is a constant in both.
    Returns (g_dx [N,2,H,W], g_dy [N,2,H,W], g_c, g_b, g_init [N,3,C,H,W])."""
    Wt = _W(dx, dy, dtype)
    b = b.to(dtype)
    c = c.to(dtype)
    grad_in = grad_out.to(dtype).clone()
    bad = ~torch.isfinite(grad_in)
    zero_out = lambda: (torch.zeros_like(dx, dtype=dtype), torch.zeros_like(dy, dtype=dtype), torch.zeros_like(c),
                        torch.zeros_like(b), torch.zeros_like(grad_in))
    if bool(bad.any()) or not bool((grad_in != 0).any()):          # :2698-2703: skip, return zeros
        return zero_out()
    sched = checkpoint_schedule(its)
    steps = step_sizes(its)
    its_eff = effective_iterations(its)
    f64 = torch.float64
    acc_c = torch.zeros(c.shape, dtype=f64)
    acc_b = torch.zeros(b.shape, dtype=f64)
    acc_x = torch.zeros(dx.shape, dtype=f64)
    acc_y = torch.zeros(dy.shape, dtype=f64)
    acc = torch.zeros_like(grad_in)
    g = None
    xbar = None
    for gi in range(its_eff - 1, -1, -1):
        t = steps[gi]
        xh = hist[gi].to(dtype)
        if gi == its_eff - 1:                                       # seed (:151-218)
            g_u, dgc, dgb = _prox_reverse(grad_in[:, 0], xh[:, 0], b, c)
            g = torch.stack([g_u, grad_in[:, 1], grad_in[:, 2]], dim=1)
            acc_c += dgc.to(f64)
            acc_b += dgb.to(f64)
            continue
        at_ckpt = gi in sched
        if exact:
            yk = ys_exact[gi + 1].to(dtype)
        elif at_ckpt:
            yk = ckpt_y[sched.index(gi)].to(dtype)
        else:
            xhm = hist[gi - 1].to(dtype)
            yk = torch.stack([rederive_y(xh[:, 0], xhm[:, 0], b, c, t), xh[:, 1], xh[:, 2]], dim=1)      # :1478-1541
        typo = (not exact) and (not at_ckpt)
        g, xbar, acc, dgc, dgb, gwx, gbx, gwy, gby = reverse_iteration(yk, g, acc, xh[:, 0], b, c, Wt, t, typo)
        acc_c += dgc.to(f64)
        acc_b += dgb.to(f64)
        acc_x += torch.cat([gwx, gbx], dim=1).to(f64)
        acc_y += torch.cat([gwy, gby], dim=1).to(f64)
    g_init = xbar.clone()
    if exact:
        ybar, gwx, gbx, gwy, gby = laplacian_transpose(ys_exact[0].to(dtype), g, Wt, False)
        g_init = ybar
        acc_x += torch.cat([gwx, gbx], dim=1).to(f64)
        acc_y += torch.cat([gwy, gby], dim=1).to(f64)
    st = state if state is not None else IdState()
    run_step = st.run / (st.run + 1.0)
    outs = {}
    gi_u = g_init[:, 0].clone()
    for key, val in (("C", acc_c), ("X", acc_x), ("Y", acc_y), ("B", acc_b), ("I", gi_u)):
        g2, av = check_grad_update(val, st.av[key])
        g2, st.av[key] = update_correct_av_step(st.run, av, st.av[key], g2, run_step)
        outs[key] = g2
    st.run += 1
    g_init = g_init.clone()
    g_init[:, 0] = outs["I"].to(dtype)          # only the primary planes pass the sanitiser (:3014-3021)
    L = Wt.L32.to(dtype)
    g_c = (outs["C"] * GLOBAL_G_MULT).to(dtype)
    g_b = (outs["B"] * GLOBAL_G_MULT).to(dtype)
    g_dx = (outs["X"] * GLOBAL_G_MULT).to(dtype) * L
    g_dy = (outs["Y"] * GLOBAL_G_MULT).to(dtype) * L
    return g_dx, g_dy, g_c, g_b, g_init


def tgv_forward_exact_ys(dx, dy, c, b, init, its: int, dtype=torch.float64):
    """All momentum iterates y_0 .. y_{its_eff} (for exact=True)."""
    Wt = _W(dx, dy, dtype)
    b = b.to(dtype); c = c.to(dtype)
    x = init.to(dtype).clone(); y = init.to(dtype).clone()
    steps = step_sizes(its)
    ys = [y.clone()]
    for g in range(effective_iterations(its)):
        y, x, _ = forward_iteration(y, x, b, c, Wt, steps[g])
        ys.append(y.clone())
    return ys
