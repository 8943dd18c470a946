"""TGV-FISTA layer: oracle pins (autograd in exact mode, golden vectors from the reference's own kernels) and GPU parity
through the C ABI."""
import os

import numpy as np
import pytest
import torch

from customnetworklayers_b200.synthetic import make_tgv_inputs
from oracle import tgv_ref as G
from tests.parity import REL_TOL, assert_close, rel_errors

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tgv_reference_cuda.npz")
NAMES = ("g_dx", "g_dy", "g_c", "g_b", "g_init")


def _golden_cases():
    z = np.load(GOLDEN)
    for i in range(int(z["n_cases"])):
        I = {k: torch.from_numpy(z[f"case{i}_{k}"]) for k in ("dx", "dy", "c", "b", "init", "grad")}
        out = {k: torch.from_numpy(z[f"case{i}_{k}"]) for k in ("sol",) + NAMES}
        yield i, int(z[f"case{i}_its"]), I, out


def test_lipschitz_constant():
    I = make_tgv_inputs(2, 1, 9, 11, seed=1)
    L = G.lipschitz_inverse(I["dx"], I["dy"])
    # alpha0 = 1, alpha1 = 2: every per-pixel bound is at most 4*2*2 + 3 = 19 < 32, so L = 1/(32 + 0.01) in fp32
    assert L.shape == (2, 1, 1, 1) and torch.all(L == torch.tensor(1.0 / np.float32(32.01), dtype=torch.float32))
    big = I["dx"].clone(); big[0, 1] = 20.0
    L2 = G.lipschitz_inverse(big, I["dy"])
    assert float(L2[0]) < float(L[0]) and float(L2[1]) == float(L[1])


@pytest.mark.parametrize("cfg", [(1, 2, 10, 12, 8), (2, 1, 7, 9, 6), (1, 3, 8, 8, 12)])
def test_exact_reverse_sweep_matches_autograd(cfg):
    n, ch, h, w, its = cfg
    I = {k: v.double() for k, v in make_tgv_inputs(n, ch, h, w, seed=5).items()}
    I["init"][:, 1:] = 0.1 * I["grad"][:, 1:]
    leaves = {k: I[k].clone().requires_grad_(True) for k in ("dx", "dy", "c", "b", "init")}
    Lfix = G.lipschitz_inverse(I["dx"], I["dy"])
    Wt = G._W(leaves["dx"], leaves["dy"], torch.float64, L=Lfix)
    x = y = leaves["init"]
    st = G.step_sizes(its)
    for g in range(G.effective_iterations(its)):
        y, x, _ = G.forward_iteration(y, x, leaves["b"], leaves["c"], Wt, st[g])
    (x * I["grad"]).sum().backward()
    sol, hist, cky, _, _ = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
    assert torch.equal(sol, x.detach())
    ys = G.tgv_forward_exact_ys(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
    gdx, gdy, gc, gb, gi = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], I["grad"], its, hist, cky, exact=True, ys_exact=ys)
    s = G.GLOBAL_G_MULT * G.LOCAL_GX_MULT
    for name, a, ref in (("init", gi, leaves["init"].grad), ("b", gb / G.GLOBAL_G_MULT, leaves["b"].grad),
                         ("c", gc / s, leaves["c"].grad), ("dx", gdx / s, leaves["dx"].grad), ("dy", gdy / s, leaves["dy"].grad)):
        assert float((a - ref).abs().max()) <= 1e-7 * max(1.0, float(ref.abs().max())), name


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32], ids=["fp64", "fp32"])
def test_oracle_reproduces_reference_kernel_outputs(dtype):
    for i, its, I, out in _golden_cases():
        sol, hist, cky, _, _ = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], its, dtype)
        grads = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], I["grad"], its, hist, cky, dtype)
        assert_close(sol, out["sol"], f"case {i} solution")
        for name, g in zip(NAMES, grads):
            assert_close(g, out[name], f"case {i} {name}")


def test_reference_approximations_are_visible_in_the_golden_vectors():
    """Against the reference kernels' outputs the exact adjoint is off by orders of magnitude more than the
    transcription: the comparison above is sensitive to what was transcribed."""
    for i, its, I, out in _golden_cases():
        if its < 10:
            continue
        sol, hist, cky, _, _ = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
        ys = G.tgv_forward_exact_ys(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
        compat = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], I["grad"], its, hist, cky)
        exact = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], I["grad"], its, hist, cky, exact=True, ys_exact=ys)
        for name, a, e in zip(NAMES[:4], compat, exact):
            ec, ee = rel_errors(a, out[name])[1], rel_errors(e, out[name])[1]
            assert ec < 1e-4 and ee > 20 * ec, (name, ec, ee)


def test_zero_or_nonfinite_upstream_gradient_returns_zeros():
    I = make_tgv_inputs(1, 1, 8, 8, seed=2)
    sol, hist, cky, _, _ = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], 4)
    z = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], torch.zeros_like(I["grad"]), 4, hist, cky)
    assert all(float(t.abs().max()) == 0 for t in z)
    g = I["grad"].clone(); g[0, 1, 0, 2, 3] = float("nan")
    z = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], g, 4, hist, cky)
    assert all(float(t.abs().max()) == 0 for t in z)


# ---------------------------------------------------------------------------------------------------------------
def _run_cuda(ext, D, its, pid, n, ch, h, w):
    flat = lambda t: t.reshape(n, 3 * ch, h, w)
    sol = ext.forward(D["dx"], D["dy"], D["c"], D["b"], flat(D["init"]), its, pid)[0]
    hist, cky, L = ext.read_history(pid, flat(D["init"]), its)
    grads = ext.backward(flat(D["grad"]), D["dx"], D["dy"], D["c"], D["b"], its, pid)
    torch.cuda.synchronize()
    five = lambda t: t.reshape(t.shape[:-3] + (3, ch, h, w))
    return five(sol), five(hist), five(cky), L, grads[:4] + [five(grads[4])]


# widths divisible by 4 run the register-tiled kernels (tiles of 7 x 120 pixels), the others the scalar ones
GPU_CASES = [(1, 1, 1, 1, 2), (1, 2, 5, 37, 4), (1, 1, 29, 3, 6), (2, 2, 40, 72, 20), (1, 3, 17, 33, 21), (1, 2, 96, 320, 20),
             (1, 2, 64, 96, 50), (1, 1, 3, 4, 2), (2, 3, 9, 124, 5), (1, 1, 15, 244, 6)]


@pytest.mark.gpu
@pytest.mark.parametrize("case", GPU_CASES, ids=lambda c: "n%d_c%d_%dx%d_its%d" % c)
def test_cuda_forward_history_and_reverse_sweep_match_oracle(case):
    from customnetworklayers_b200 import tgvInpaint_cuda_ext as ext
    n, ch, h, w, its = case
    I = make_tgv_inputs(n, ch, h, w, seed=50 + h + w)
    I["init"][:, 1:] = 0.1 * I["grad"][:, 1:]
    D = {k: v.cuda() for k, v in I.items()}
    ext.release(3)
    ext.set_option(3, 1, 0)
    sol, hist, cky, L, grads = _run_cuda(ext, D, its, 3, n, ch, h, w)
    r_sol, r_hist, r_cky, _, r_L = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
    assert torch.equal(L.cpu(), r_L.reshape(-1)), "1/Lipschitz must be bit-exact"
    assert_close(sol, r_sol, "solution")
    assert_close(hist, r_hist, "history")
    assert_close(cky, r_cky, "checkpointed y")
    # reverse sweep on exactly the iterates the device stored (it is discontinuous at the Huber thresholds)
    ref = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], I["grad"], its, hist.cpu(), cky.cpu())
    for name, g, r in zip(NAMES, grads, ref):
        assert_close(g, r, name)


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(2, 2, 40, 72, 20), (2, 3, 9, 124, 5), (1, 1, 15, 244, 6), (3, 1, 23, 128, 9)],
                         ids=lambda c: "n%d_c%d_%dx%d_its%d" % c)
def test_persistent_kernels_match_oracle(case, monkeypatch):
    """The persistent, pipelined kernels normally serve launches of thousands of tiles; forced here."""
    from customnetworklayers_b200 import tgvInpaint_cuda_ext as ext
    monkeypatch.setenv("CNL_TGV_PIPELINE_MIN_TILES", "1")
    monkeypatch.setenv("CNL_TGV_REV_PIPELINE_MIN_TILES", "1")
    n, ch, h, w, its = case
    I = make_tgv_inputs(n, ch, h, w, seed=11 + h + w)
    I["init"][:, 1:] = 0.1 * I["grad"][:, 1:]
    D = {k: v.cuda() for k, v in I.items()}
    ext.release(3)
    ext.set_option(3, 1, 0)
    sol, hist, cky, L, grads = _run_cuda(ext, D, its, 3, n, ch, h, w)
    r_sol, r_hist, r_cky, _, r_L = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
    assert_close(sol, r_sol, "solution")
    assert_close(hist, r_hist, "history")
    assert_close(cky, r_cky, "checkpoints")
    ref = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], I["grad"], its, hist.cpu(), cky.cpu())
    for name, g, r in zip(NAMES, grads, ref):
        assert_close(g, r, name)
    monkeypatch.setenv("CNL_TGV_PIPELINE_MIN_TILES", "-1")
    monkeypatch.setenv("CNL_TGV_REV_PIPELINE_MIN_TILES", "-1")
    sol2, _, _, _, grads2 = _run_cuda(ext, D, its, 3, n, ch, h, w)
    assert torch.equal(sol, sol2), "both forward kernels do the same arithmetic"
    for name, a, b in zip(NAMES, grads, grads2):
        assert torch.equal(a, b), name + ": both reverse kernels do the same arithmetic"


@pytest.mark.gpu
def test_cuda_reproduces_reference_kernel_outputs():
    from customnetworklayers_b200 import tgvInpaint_cuda_ext as ext
    for i, its, I, out in _golden_cases():
        n, ch, h, w = I["b"].shape
        D = {k: v.cuda() for k, v in I.items()}
        ext.release(4)
        ext.set_option(4, 1, 0)
        sol, _, _, _, grads = _run_cuda(ext, D, its, 4, n, ch, h, w)
        assert_close(sol, out["sol"], f"case {i} solution")
        for name, g in zip(NAMES, grads):
            assert_close(g, out[name], f"case {i} {name}")


@pytest.mark.gpu
def test_cuda_batch_equals_single_calls_and_skip_rule():
    from customnetworklayers_b200 import tgvInpaint_cuda_ext as ext
    n, ch, h, w, its = 3, 2, 30, 44, 8
    I = make_tgv_inputs(n, ch, h, w, seed=77)
    I["dx"][1, 1] = 30.0          # a different Lipschitz constant for the second image
    D = {k: v.cuda() for k, v in I.items()}
    for pid in (5, 6):
        ext.release(pid)
        ext.set_option(pid, 1, 0)
    sol, _, _, L, grads = _run_cuda(ext, D, its, 5, n, ch, h, w)
    assert float(L[1]) < float(L[0])
    for i in range(n):
        Di = {k: v[i:i + 1].contiguous() for k, v in D.items()}
        s1, _, _, _, g1 = _run_cuda(ext, Di, its, 6, 1, ch, h, w)
        assert torch.equal(s1[0], sol[i])
        for name, a, b in zip(NAMES, g1, grads):
            assert torch.equal(a[0], b[i]), name
    # an identically zero or non-finite upstream gradient yields all-zero gradients
    flat = lambda t: t.reshape(n, 3 * ch, h, w)
    ext.forward(D["dx"], D["dy"], D["c"], D["b"], flat(D["init"]), its, 5)
    z = ext.backward(torch.zeros_like(flat(D["grad"])), D["dx"], D["dy"], D["c"], D["b"], its, 5)
    assert all(float(t.abs().max()) == 0 for t in z)
    bad = flat(D["grad"]).clone(); bad[0, 0, 1, 1] = float("inf")
    z = ext.backward(bad, D["dx"], D["dy"], D["c"], D["b"], its, 5)
    assert all(float(t.abs().max()) == 0 for t in z)


@pytest.mark.gpu
def test_tgv_layer_api():
    from customnetworklayers_b200.TGVInpainting import TGVInpaint
    ch, h, w, its = 2, 24, 32, 6
    I = make_tgv_inputs(1, ch, h, w, seed=9)
    hwc = lambda t: t[0].permute(1, 2, 0).contiguous().cuda()
    leaves = [hwc(I["dx"]), hwc(I["dy"]), hwc(I["c"]), hwc(I["b"]), hwc(I["init"].reshape(1, 3 * ch, h, w))]
    leaves = [t.requires_grad_(True) for t in leaves]
    out = TGVInpaint("cuda", its, pid=7)(*leaves)
    assert out.shape == (h, w, 3 * ch)
    out.backward(hwc(I["grad"].reshape(1, 3 * ch, h, w)))
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in leaves)
    r_sol, *_ = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
    assert_close(out.permute(2, 0, 1).reshape(1, 3, ch, h, w), r_sol, "layer output")


@pytest.mark.gpu
def test_full_size_properties():
    """Size-independent properties at the secondary benchmark's full size (batch 8, 2x436x1024, 100 iterations):
    batch independence and linearity of the reverse sweep in the upstream gradient."""
    from customnetworklayers_b200 import tgvInpaint_cuda_ext as ext
    n, ch, h, w, its = 8, 2, 436, 1024, 100
    D = {k: v.cuda() for k, v in make_tgv_inputs(n, ch, h, w, seed=99).items()}
    flat = lambda t: t.reshape(t.shape[0], 3 * ch, h, w)
    for pid in (7, 8):
        ext.release(pid)
        ext.set_option(pid, 1, 0)
    try:
        sol = ext.forward(D["dx"], D["dy"], D["c"], D["b"], flat(D["init"]), its, 7)[0]
        g1 = ext.backward(flat(D["grad"]), D["dx"], D["dy"], D["c"], D["b"], its, 7)
        assert all(bool(torch.isfinite(t).all()) for t in (sol,) + tuple(g1))
        g2 = ext.backward(2.0 * flat(D["grad"]), D["dx"], D["dy"], D["c"], D["b"], its, 7)
        for name, a, b in zip(NAMES, g1, g2):
            assert float((2.0 * a - b).abs().max()) <= 1e-30, name + ": backward(2 g) != 2 backward(g)"
        k = 3
        one = {key: D[key][k:k + 1].contiguous() for key in D}
        sol_k = ext.forward(one["dx"], one["dy"], one["c"], one["b"], flat(one["init"]), its, 8)[0]
        gk = ext.backward(flat(one["grad"]), one["dx"], one["dy"], one["c"], one["b"], its, 8)
        torch.cuda.synchronize()
        assert torch.equal(sol_k[0], sol[k])
        for name, a, b in zip(NAMES, g1, gk):
            assert torch.equal(a[k], b[0]), name + ": batch member differs from the single call"
    finally:
        for pid in (7, 8):
            ext.set_option(pid, 1, 1)
            ext.release(pid)


@pytest.mark.gpu
def test_widths_and_pointers_that_need_staging():
    """Rows that are not a multiple of four floats and misaligned tensors run the register-tiled kernels on zero-padded
    copies: oracle parity on a 1242-pixel-wide problem, and the bits of the aligned call for a misaligned one."""
    from customnetworklayers_b200 import tgvInpaint_cuda_ext as ext
    n, ch, h, w, its = 2, 2, 20, 1242, 6
    I = make_tgv_inputs(n, ch, h, w, seed=321)
    I["init"][:, 1:] = 0.1 * I["grad"][:, 1:]
    D = {k: v.cuda() for k, v in I.items()}
    ext.release(3)
    ext.set_option(3, 1, 0)
    sol, hist, cky, L, grads = _run_cuda(ext, D, its, 3, n, ch, h, w)
    r_sol, r_hist, r_cky, _, r_L = G.tgv_forward_history(I["dx"], I["dy"], I["c"], I["b"], I["init"], its)
    assert_close(sol, r_sol, "solution")
    assert_close(hist, r_hist, "history")
    ref = G.tgv_backward(I["dx"], I["dy"], I["c"], I["b"], I["grad"], its, hist.cpu(), cky.cpu())
    for name, g, r in zip(NAMES, grads, ref):
        assert_close(g, r, name)

    n, ch, h, w, its = 1, 2, 16, 64, 8
    I = make_tgv_inputs(n, ch, h, w, seed=322)
    D = {k: v.cuda() for k, v in I.items()}
    sol_a, _, _, _, g_a = _run_cuda(ext, D, its, 3, n, ch, h, w)

    def shifted(t):              # same values, storage offset of one float
        buf = torch.empty(t.numel() + 1, device=t.device, dtype=t.dtype)
        view = buf[1:].view(t.shape)
        view.copy_(t)
        return view
    U = {k: shifted(v) for k, v in D.items()}
    sol_u, _, _, _, g_u = _run_cuda(ext, U, its, 3, n, ch, h, w)
    assert torch.equal(sol_a, sol_u)
    for name, a, b in zip(NAMES, g_a, g_u):
        assert torch.equal(a, b), name
    ext.set_option(3, 1, 1)
    ext.release(3)
