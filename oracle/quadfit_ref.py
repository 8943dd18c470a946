"""CPU restatement of the reference's differentiable quadratic fit (cudaQuadFit/cudaCode/quadFit.cu).
TEST INFRASTRUCTURE ONLY.

Forward (kQuadFitFlow, quadFit.cu:14-136): for every pixel, the displaced location (w + flow_x, h + flow_y) is
rounded to the nearest pixel of the second image; the correlation of the pixel's feature vector with the features
at that location and its four neighbours gives a 5-point stencil; a concave quadratic is fitted per axis and its
maximiser (fx, fy) and the fitted score are returned as [N,3,H,W].  Pixels whose displaced location leaves the
image keep (0,0,0).  Backward (kQuadFitFlowGrad, :142-297): gradients w.r.t. both feature maps (none w.r.t. flow).

The float / double promotions of the reference's expressions are reproduced (they decide the rounding of the
integer location and of the validity tests).  Pinned by golden vectors from the reference's own kernels."""
from __future__ import annotations

import numpy as np

f32 = np.float32
f64 = np.float64


def _locate(flow, H, W):
    n = flow.shape[0]
    ww = np.arange(W, dtype=f32).reshape(1, 1, W)
    hh = np.arange(H, dtype=f32).reshape(1, H, 1)
    idx = (ww + flow[:, 0].astype(f32)).astype(f32)                    # :31
    idy = (hh + flow[:, 1].astype(f32)).astype(f32)                    # :32
    inside = ~((idx > W - 1) | (idx < 0) | (idy > H - 1) | (idy < 0))  # :35
    iidx = np.floor(idx.astype(f64) + 0.5).astype(np.int64)            # :46, double
    iidy = np.floor(idy.astype(f64) + 0.5).astype(np.int64)
    iidx = np.where(inside, iidx, 0)
    iidy = np.where(inside, iidy, 0)
    return inside, iidx, iidy


def fit_from_costs(c00, c0p, cp0, c0m, cm0, interior_x, interior_y):
    """The per-axis fit (quadFit.cu:74-134) on fp32 cost arrays. Returns dict of fp32 arrays."""
    ax = (0.5 * ((c0p + c0m).astype(f32).astype(f64) - 2.0 * c00.astype(f64))).astype(f32)      # :74
    ay = (0.5 * ((cp0 + cm0).astype(f32).astype(f64) - 2.0 * c00.astype(f64))).astype(f32)
    bx = (0.5 * (c0p - c0m).astype(f32).astype(f64)).astype(f32)
    by = (0.5 * (cp0 - cm0).astype(f32).astype(f64)).astype(f32)
    vx = (ax < 0) & ((ax * ax).astype(f32).astype(f64) >= 0.25 * bx.astype(f64) * bx.astype(f64)) & interior_x   # :82-88
    vy = (ay < 0) & ((ay * ay).astype(f32).astype(f64) >= 0.25 * by.astype(f64) * by.astype(f64)) & interior_y
    with np.errstate(divide="ignore", invalid="ignore"):
        fx = np.where(vx, (-0.5 * bx.astype(f64) / ax.astype(f64)), 0.0).astype(f32)             # :92
        fy = np.where(vy, (-0.5 * by.astype(f64) / ay.astype(f64)), 0.0).astype(f32)
    score = (ax * fx * fx + bx * fx + c00 + ay * fy * fy + by * fy).astype(f32)                  # :133
    return {"ax": ax, "ay": ay, "bx": bx, "by": by, "vx": vx, "vy": vy, "fx": fx, "fy": fy, "score": score}


def _stencil(feat0, feat1, inside, iidx, iidy):
    n, c, H, W = feat0.shape
    xm, xp = np.maximum(iidx - 1, 0), np.minimum(iidx + 1, W - 1)
    ym, yp = np.maximum(iidy - 1, 0), np.minimum(iidy + 1, H - 1)
    ni = np.arange(n).reshape(n, 1, 1, 1)
    ci = np.arange(c).reshape(1, c, 1, 1)
    g = lambda yy, xx: feat1[ni, ci, yy[:, None], xx[:, None]]
    return (g(iidy, iidx), g(iidy, xp), g(yp, iidx), g(iidy, xm), g(ym, iidx)), (xm, xp, ym, yp)


def quadfit_forward(feat0, feat1, flow):
    """feat0, feat1 [N,C,H,W], flow [N,>=2,H,W] (fp32) -> (out [N,3,H,W] fp32, iidx, iidy int arrays, inside mask)."""
    feat0 = np.asarray(feat0, f32); feat1 = np.asarray(feat1, f32); flow = np.asarray(flow, f32)
    n, c, H, W = feat0.shape
    inside, iidx, iidy = _locate(flow, H, W)
    (I00, I0p, Ip0, I0m, Im0), _ = _stencil(feat0, feat1, inside, iidx, iidy)
    costs = []
    for I2 in (I00, I0p, Ip0, I0m, Im0):
        acc = np.zeros((n, H, W), dtype=f32)
        for cc in range(c):                                 # sequential fp32 accumulation (:62-70)
            acc = (acc + feat0[:, cc] * I2[:, cc]).astype(f32)
        costs.append(acc)
    fit = fit_from_costs(*costs, (iidx < W - 1) & (iidx > 0), (iidy < H - 1) & (iidy > 0))
    out = np.zeros((n, 3, H, W), dtype=f32)
    out[:, 0] = np.where(inside, fit["fx"], 0)
    out[:, 1] = np.where(inside, fit["fy"], 0)
    out[:, 2] = np.where(inside, fit["score"], 0)
    return out, iidx, iidy, inside


def _fit_gradient_coeffs(fit, gfx, gfy, gs):
    """Coefficients of d loss / d (c00, c0p, c0m, cp0, cm0) (quadFit.cu:245-281), in float64."""
    vx, vy = fit["vx"], fit["vy"]
    ax, ay, fx, fy = (fit[k].astype(f64) for k in ("ax", "ay", "fx", "fy"))
    with np.errstate(divide="ignore", invalid="ignore"):
        dfx_dbx = np.where(vx, -1.0 / (2.0 * ax), 0.0).astype(f32).astype(f64)
        dfx_dax = np.where(vx, -fx / ax, 0.0).astype(f32).astype(f64)
        dfy_dby = np.where(vy, -1.0 / (2.0 * ay), 0.0).astype(f32).astype(f64)
        dfy_day = np.where(vy, -fy / ay, 0.0).astype(f32).astype(f64)
    ds_dax = np.where(vx, fx * fx, 0.0).astype(f32).astype(f64)
    ds_dbx = np.where(vx, fx, 0.0)
    ds_day = np.where(vy, fy * fy, 0.0).astype(f32).astype(f64)
    ds_dby = np.where(vy, fy, 0.0)
    ds_dc = np.where(vx | vy, 1.0, 0.0)
    gfx, gfy, gs = gfx.astype(f64), gfy.astype(f64), gs.astype(f64)
    Ax = gfx * dfx_dax + gs * ds_dax
    Bx = gfx * dfx_dbx + gs * ds_dbx
    Ay = gfy * dfy_day + gs * ds_day
    By = gfy * dfy_dby + gs * ds_dby
    any_valid = vx | vy
    k00 = np.where(any_valid, 0.5 * (-2.0 * Ax - 2.0 * Ay + 2.0 * gs * ds_dc), gs)      # else-branch: score passes through
    k0p = np.where(any_valid, 0.5 * (Ax + Bx), 0.0)
    k0m = np.where(any_valid, 0.5 * (Ax - Bx), 0.0)
    kp0 = np.where(any_valid, 0.5 * (Ay + By), 0.0)
    km0 = np.where(any_valid, 0.5 * (Ay - By), 0.0)
    return k00, k0p, k0m, kp0, km0


def quadfit_backward(feat0, feat1, flow, grad):
    """grad [N,3,H,W] -> (g_feat0, g_feat1) [N,C,H,W] float32 (accumulated in float64 before the final cast)."""
    feat0 = np.asarray(feat0, f32); feat1 = np.asarray(feat1, f32); flow = np.asarray(flow, f32); grad = np.asarray(grad, f32)
    n, c, H, W = feat0.shape
    out, iidx, iidy, inside = quadfit_forward(feat0, feat1, flow)
    (I00, I0p, Ip0, I0m, Im0), (xm, xp, ym, yp) = _stencil(feat0, feat1, inside, iidx, iidy)
    costs = []
    for I2 in (I00, I0p, Ip0, I0m, Im0):
        acc = np.zeros((n, H, W), dtype=f32)
        for cc in range(c):
            acc = (acc + feat0[:, cc] * I2[:, cc]).astype(f32)
        costs.append(acc)
    fit = fit_from_costs(*costs, (iidx < W - 1) & (iidx > 0), (iidy < H - 1) & (iidy > 0))
    k00, k0p, k0m, kp0, km0 = _fit_gradient_coeffs(fit, grad[:, 0], grad[:, 1], grad[:, 2])
    m = inside.astype(f64)
    k00, k0p, k0m, kp0, km0 = (k * m for k in (k00, k0p, k0m, kp0, km0))
    g0 = (I00.astype(f64) * k00[:, None] + I0p * k0p[:, None] + I0m * k0m[:, None] + Ip0 * kp0[:, None] + Im0 * km0[:, None])
    g1 = np.zeros((n, c, H, W), dtype=f64)
    ni = np.broadcast_to(np.arange(n).reshape(n, 1, 1, 1), (n, c, H, W))
    ci = np.broadcast_to(np.arange(c).reshape(1, c, 1, 1), (n, c, H, W))
    f0 = feat0.astype(f64)
    bc = lambda a: np.broadcast_to(a[:, None], (n, c, H, W))
    for yy, xx, k in ((iidy, iidx, k00), (iidy, xp, k0p), (iidy, xm, k0m), (yp, iidx, kp0), (ym, iidx, km0)):
        np.add.at(g1, (ni, ci, bc(yy), bc(xx)), f0 * k[:, None])
    return g0.astype(f32), g1.astype(f32)


def quadfit_from_cost_forward(cost5):
    """cost5 [N,5,H,W] = (c00, c0p, cp0, c0m, cm0) of a correlation to MAXIMISE -> out [N,3,H,W]; no border tests."""
    cost5 = np.asarray(cost5, f32)
    t = np.ones(cost5.shape[0:1] + cost5.shape[2:], dtype=bool)
    fit = fit_from_costs(cost5[:, 0], cost5[:, 1], cost5[:, 2], cost5[:, 3], cost5[:, 4], t, t)
    return np.stack([fit["fx"], fit["fy"], fit["score"]], axis=1).astype(f32)


def quadfit_from_cost_backward(cost5, grad):
    cost5 = np.asarray(cost5, f32); grad = np.asarray(grad, f32)
    t = np.ones(cost5.shape[0:1] + cost5.shape[2:], dtype=bool)
    fit = fit_from_costs(cost5[:, 0], cost5[:, 1], cost5[:, 2], cost5[:, 3], cost5[:, 4], t, t)
    k00, k0p, k0m, kp0, km0 = _fit_gradient_coeffs(fit, grad[:, 0], grad[:, 1], grad[:, 2])
    return np.stack([k00, k0p, kp0, k0m, km0], axis=1).astype(f32)
