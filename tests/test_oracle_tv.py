"""Pins the CPU oracle: forward against an independent per-pixel loop restatement, the reverse sweep against
torch.autograd of an independently written differentiable forward, and the host-side schedules."""
import math

import numpy as np
import pytest
import torch

from oracle import tv_ref as R


def test_checkpoint_schedules():
    # values follow from floor(i*sqrt(its)*0.5)*2, i < floor(sqrt(its))   (TVInpaintFista.cu:1499-1504)
    assert R.checkpoint_schedule(20) == [0, 4, 8, 12]
    assert R.checkpoint_schedule(50) == [0, 6, 14, 20, 28, 34, 42]
    assert R.checkpoint_schedule(100) == list(range(0, 100, 10))
    assert R.checkpoint_schedule(2) == [0]
    for its in range(2, 200):
        s = R.checkpoint_schedule(its)
        assert s[0] == 0 and all(a < b for a, b in zip(s, s[1:])) and all(v % 2 == 0 for v in s)
        assert s[-1] < R.effective_iterations(its)


def test_step_sizes():
    st = R.step_sizes(6)
    assert st[0] == 0.0
    t1 = (1 + math.sqrt(5)) / 2
    t2 = (1 + math.sqrt(1 + 4 * t1 * t1)) / 2
    assert abs(st[1] - (t1 - 1) / t2) < 1e-7
    assert all(0 <= s < 1 for s in st) and all(a <= b for a, b in zip(st, st[1:]))


@pytest.mark.parametrize("shape", [(1, 5, 7), (2, 6, 5), (3, 1, 9), (1, 8, 1), (1, 1, 1)])
def test_forward_iteration_matches_pixel_loops(shape):
    C, H, W = shape
    inp = R.make_inputs(1, C, H, W, seed=7)
    gen = torch.Generator().manual_seed(3)
    y = (torch.rand(1, C, H, W, generator=gen, dtype=torch.float64) * 4 - 2)
    xp = (torch.rand(1, C, H, W, generator=gen, dtype=torch.float64) * 4 - 2)
    b = inp["b"].double() * 0.1
    wts = R._prepare_weights(inp["wx"], inp["wy"], torch.float64)
    yn, xn, x05 = R.forward_iteration(y, xp, b, inp["c"].double(), wts, 0.37)
    yl, xl, x05l = R.forward_iteration_loops(y[0].numpy(), xp[0].numpy(), b[0].numpy(), inp["c"][0, 0].double().numpy(),
                                             inp["wx"][0, 0].double().numpy(), inp["wy"][0, 0].double().numpy(), 0.37)
    np.testing.assert_allclose(x05[0].numpy(), x05l, rtol=0, atol=1e-12)
    np.testing.assert_allclose(xn[0].numpy(), xl, rtol=0, atol=1e-12)
    np.testing.assert_allclose(yn[0].numpy(), yl, rtol=0, atol=1e-12)


# ---- an independently written differentiable forward (flux / divergence form) -------------------------------
def _diff_forward(wx, wy, c, b, init, its):
    d = R.HUBER_DELTA
    N, C, H, W = b.shape
    mx = torch.ones(1, 1, H, W, dtype=b.dtype)
    mx[..., -1] = 0
    my = torch.ones(1, 1, H, W, dtype=b.dtype)
    my[..., -1, :] = 0
    wxs = wx * R.LIPSCHITZ_INV * mx
    wys = wy * R.LIPSCHITZ_INV * my
    steps = R.step_sizes(its)
    x = init
    y = init
    pad = torch.nn.functional.pad
    for g in range(R.effective_iterations(its)):
        d1 = y - pad(y[..., :, 1:], (0, 1))          # y[p] - y[p+x]
        d2 = y - pad(y[..., 1:, :], (0, 0, 0, 1))    # y[p] - y[p+y]
        A = wxs * d1 * d1 + wys * d2 * d2
        big = A > d * d
        s = torch.where(big, d / torch.sqrt(torch.where(big, A, torch.ones_like(A))), torch.ones_like(A))
        fx = s * wxs * d1
        fy = s * wys * d2
        x05 = y - fx - fy + pad(fx[..., :, :-1], (1, 0)) + pad(fy[..., :-1, :], (0, 0, 1, 0))
        xq = (c * b + x05) / (1 + c)
        xn = torch.where(x05 - c > 1 + b, x05 - c, torch.where(x05 + c < b - 1, x05 + c, xq))
        y = xn + steps[g] * (xn - x)
        x = xn
    return x


def _inputs64(n, ch, h, w, seed, scale=1.0):
    inp = R.make_inputs(n, ch, h, w, seed=seed)
    out = {k: v.double() for k, v in inp.items()}
    out["b"] = out["b"] * scale
    out["init"] = out["b"].clone() + 0.05 * out["grad"]
    return out


@pytest.mark.parametrize("cfg", [(1, 2, 9, 11, 8), (2, 1, 7, 6, 20), (1, 3, 12, 10, 26)])
def test_forward_matches_differentiable_restatement(cfg):
    n, ch, h, w, its = cfg
    I = _inputs64(n, ch, h, w, seed=11)
    sol, _ = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    sol2 = _diff_forward(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    assert torch.allclose(sol, sol2, rtol=0, atol=1e-10)


@pytest.mark.parametrize("cfg", [(1, 2, 9, 11, 8, 1.0), (2, 1, 7, 6, 20, 0.2), (1, 3, 12, 10, 26, 1.0), (1, 2, 6, 6, 2, 1.0)])
def test_exact_backward_matches_autograd(cfg):
    """exact=True removes the reference's approximations; what is left (Laplacian transpose, Huber-weight
    derivative, prox Jacobian, momentum reverse, weight/confidence/rhs gradients) must equal autograd."""
    n, ch, h, w, its, scale = cfg
    I = _inputs64(n, ch, h, w, seed=5, scale=scale)
    leaves = {k: I[k].clone().requires_grad_(True) for k in ("wx", "wy", "c", "b", "init")}
    sol = _diff_forward(leaves["wx"], leaves["wy"], leaves["c"], leaves["b"], leaves["init"], its)
    (sol * I["grad"]).sum().backward()
    _, ckpts = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    gwx, gwy, gc, gb, gi = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ckpts, exact=True)
    s2 = R.GLOBAL_G_MULT * R.LOCAL_GC_MULT
    mx = torch.ones_like(gwx); mx[..., -1] = 0
    my = torch.ones_like(gwy); my[..., -1, :] = 0
    def close(a, ref):
        return float((a - ref).abs().max()) <= 1e-9 * max(1.0, float(ref.abs().max()))
    assert close(gi, leaves["init"].grad)
    assert close(gb / (R.GLOBAL_G_MULT * R.LOCAL_GB_MULT), leaves["b"].grad)
    assert close(gc / s2, leaves["c"].grad)
    assert close(gwx / (R.GLOBAL_G_MULT * R.LOCAL_GX_MULT), leaves["wx"].grad * mx)
    assert close(gwy / (R.GLOBAL_G_MULT * R.LOCAL_GX_MULT), leaves["wy"].grad * my)


def test_ref_compat_backward_is_close_to_exact_but_not_equal():
    """The reference's approximations are small corrections: same order of magnitude, measurably different."""
    I = _inputs64(1, 2, 16, 20, seed=9)
    its = 20
    _, ckpts = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    ex = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ckpts, exact=True)
    rc = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ckpts, exact=False)
    for a, r in zip(rc[:4], ex[:4]):
        rel = float((a - r).norm() / r.norm())
        assert rel < 0.8
    assert any(float((a - r).abs().max()) > 0 for a, r in zip(rc, ex))


def test_id_slots_and_errors():
    ref = R.TVInpaintFistaRef()
    I = _inputs64(1, 2, 8, 8, seed=2)
    with pytest.raises(ValueError):
        ref.forward(I["wx"], I["wy"], I["c"], I["b"], I["init"], 4, 10)
    with pytest.raises(RuntimeError):
        ref.backward(I["grad"], I["wx"], I["wy"], I["c"], I["b"], 4, 3)
    s0 = ref.forward(I["wx"], I["wy"], I["c"], I["b"], I["init"], 4, 0)
    s1 = ref.forward(I["wx"], I["wy"], I["c"], I["b"] * 0.5, I["init"], 6, 1)
    g0 = ref.backward(I["grad"], I["wx"], I["wy"], I["c"], I["b"], 4, 0)
    g1 = ref.backward(I["grad"], I["wx"], I["wy"], I["c"], I["b"] * 0.5, 6, 1)
    assert s0.shape == s1.shape and len(g0) == len(g1) == 5
    assert ref.ids[0].run == 1 and ref.ids[1].run == 1 and ref.ids[2].run == 0


def test_odd_its_runs_even_count():
    I = _inputs64(1, 1, 6, 6, seed=4)
    a, _ = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], 7)
    b6 = _diff_forward(I["wx"], I["wy"], I["c"], I["b"], I["init"], 6)
    # step table of its=7 and its=6 agree on the first six entries
    assert torch.allclose(a, b6, atol=1e-10)


def test_sanitiser_and_conditioner():
    g = torch.tensor([1.0, float("nan"), 2e7, -3.0], dtype=torch.float64)
    out, av = R.check_grad_update(g, av_current=2.0)
    assert out.tolist() == [1.0, 0.0, 0.0, -3.0]
    # after the invalid entry at i=1 the mean restarts from av_current*1000
    exp = 2000.0
    exp = (1 - 2 / 3) * 2e7 + (2 / 3) * exp
    exp = (1 - 3 / 4) * 3.0 + (3 / 4) * exp
    assert abs(av - exp) < 1e-6
    g2, st = R.update_correct_av_step(3, 100.0, 1.0, torch.ones(3), 0.75)      # run < 10: identity
    assert g2.tolist() == [1, 1, 1] and abs(st - (0.75 + 25.0)) < 1e-12
    g3, st = R.update_correct_av_step(12, 100.0, 1.0, torch.ones(3), 0.9)      # > 50x: kill
    assert g3.abs().sum() == 0 and abs(st - (0.9 + 0.1 * 10)) < 1e-12
    g4, st = R.update_correct_av_step(12, 20.0, 1.0, torch.ones(3), 0.9)       # > 10x: rescale to 10x
    assert torch.allclose(g4, torch.full((3,), 0.5))
