"""Golden vectors produced by the reference's own cudaTV kernels on a B200 (tests/golden/make_golden.py):
the CPU oracle must reproduce them (no GPU needed), and so must the CUDA path (gpu)."""
import os

import numpy as np
import pytest
import torch

from oracle import tv_ref as R
from tests.parity import assert_close

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tv_reference_cuda.npz")
NAMES = ("g_wx", "g_wy", "g_c", "g_b", "g_init")


def _cases():
    z = np.load(GOLDEN)
    for i in range(int(z["n_cases"])):
        I = {k: torch.from_numpy(z[f"case{i}_{k}"]) for k in ("wx", "wy", "c", "b", "init", "grad")}
        out = {k: torch.from_numpy(z[f"case{i}_{k}"]) for k in ("sol",) + NAMES}
        yield i, int(z[f"case{i}_its"]), I, out


def test_golden_file_is_present_and_small():
    assert os.path.exists(GOLDEN) and os.path.getsize(GOLDEN) < 1 << 20


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32], ids=["fp64", "fp32"])
def test_oracle_reproduces_reference_kernel_outputs(dtype):
    for i, its, I, out in _cases():
        sol, ck = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its, dtype)
        grads = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck, dtype)
        assert_close(sol, out["sol"], f"case {i} solution")
        for name, g in zip(NAMES, grads):
            assert_close(g, out[name], f"case {i} {name}")


@pytest.mark.gpu
def test_cuda_path_reproduces_reference_kernel_outputs():
    from customnetworklayers_b200 import tvInpaint_cuda_ext as ext
    for i, its, I, out in _cases():
        D = {k: v.cuda() for k, v in I.items()}
        ext.release(4)
        ext.set_option(4, 1, 0)
        sol = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 4)[0]
        grads = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 4)
        assert_close(sol, out["sol"], f"case {i} solution")
        for name, g in zip(NAMES, grads):
            assert_close(g, out[name], f"case {i} {name}")
