"""Pins the oracle and the CUDA path against the reference's OWN kernels (oracle/_ref/libtvref.so, the unmodified
cudaTV sources built against a small ImageUtilities stand-in).  Skipped when that library was not built."""
import pytest
import torch

from oracle import ref_cuda
from oracle import tv_ref as R
from tests.parity import REL_TOL, assert_close, rel_errors

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libtvref.so not built")]

GRAD_NAMES = ["g_wx", "g_wy", "g_c", "g_b", "g_init"]


def _dev(I):
    return {k: v.cuda() for k, v in I.items()}


# the reference is only safe for heights % 16 == 0 and widths % 32 == 0 (it reads before its bounds check)
@pytest.mark.parametrize("case", [(1, 16, 32, 4), (2, 32, 64, 6), (2, 48, 96, 20), (3, 32, 32, 10), (2, 96, 320, 20)],
                         ids=lambda c: "c%d_%dx%d_its%d" % c)
def test_reference_kernels_agree_with_oracle_and_cuda_path(case):
    from customnetworklayers_b200 import tvInpaint_cuda_ext as ext
    ch, h, w, its = case
    I = R.make_inputs(1, ch, h, w, seed=31 + h + w + its)
    D = _dev(I)
    # --- forward: reference kernels vs fp64 oracle vs this library
    ref_sol = ref_cuda.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 1)
    o_sol, hist64, cky64 = R.tv_forward_history(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    ext.release(1)
    ext.set_option(1, 1, 0)
    my_sol = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 1)[0]
    assert_close(ref_sol, o_sol, "reference kernels vs oracle: solution")
    assert_close(my_sol, ref_sol.cpu(), "this library vs reference kernels: solution")
    # --- backward, end to end.  The reverse sweep is discontinuous at the Huber thresholds, so the bound is the
    # larger of 1e-4 and 5x the oracle's own fp32-vs-fp64 gap on these inputs (both printed).
    ref_g = ref_cuda.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 1)
    my_g = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 1)
    _, ck64 = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its, torch.float64)
    g64 = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck64, torch.float64)
    _, ck32 = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its, torch.float32)
    g32 = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck32, torch.float32)
    for name, rg, mg, o64, o32 in zip(GRAD_NAMES, ref_g, my_g, g64, g32):
        gap = rel_errors(o32, o64)
        e_ref = rel_errors(rg, o64)
        e_my = rel_errors(mg, rg.cpu())
        print(f"{name}: ref-vs-oracle64 max {e_ref[0]:.2e} l2 {e_ref[1]:.2e} | lib-vs-ref max {e_my[0]:.2e} l2 {e_my[1]:.2e}"
              f" | oracle32-vs-64 max {gap[0]:.2e} l2 {gap[1]:.2e}")
        bound = max(REL_TOL, 5.0 * gap[1])
        assert e_ref[1] <= bound, f"reference kernels vs oracle: {name} l2 {e_ref[1]:.2e} > {bound:.2e}"
        assert e_my[1] <= bound, f"this library vs reference kernels: {name} l2 {e_my[1]:.2e} > {bound:.2e}"


def test_reference_quirks_are_what_the_oracle_transcribes():
    """The exact-adjoint mode of the oracle must NOT match the reference kernels while the transcribed
    approximations do: shows that the comparison above is sensitive to the quirks."""
    ch, h, w, its = 2, 32, 64, 20
    I = R.make_inputs(1, ch, h, w, seed=77)
    D = _dev(I)
    ref_cuda.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 2)
    ref_g = ref_cuda.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 2)
    _, ck = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    compat = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck, exact=False)
    exact = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck, exact=True)
    for name, rg, a, e in zip(GRAD_NAMES, ref_g, compat, exact):
        ec = rel_errors(rg, a)[1]
        ee = rel_errors(rg, e)[1]
        print(f"{name}: vs transcription {ec:.2e}, vs exact adjoint {ee:.2e}")
        assert ec < 5e-3
        assert ee > 10 * ec
