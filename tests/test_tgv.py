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
