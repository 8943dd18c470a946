"""Weighted-median selection layer: CPU oracle pins (hand-worked cases, golden vectors from the reference's own
kernel) and GPU parity through the C ABI.  The crossing index must be bit-exact."""
import os

import numpy as np
import pytest
import torch

from customnetworklayers_b200.synthetic import make_median_volume
from oracle import median_ref as M
from tests.parity import assert_close

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "median_reference_cuda.npz")


def test_oracle_hand_worked_cases():
    # weights .2 .2 .2 .4 : running sums .2 .4 .6 -> crossing at bin 2; alpha = (1 - 2*.4 - .2) / (2*.2) = 0
    vol = np.array([0.2, 0.2, 0.2, 0.4], dtype=np.float32).reshape(1, 1, 1, 4)
    out, idx = M.median_forward(vol)
    assert idx[0, 0, 0] == 2 and abs(out[0, 0, 0, 0] - 2.0) < 1e-6 and abs(out[0, 1, 0, 0] - 0.2) < 1e-7
    # all mass in bin 0: crossing at 0 with alpha = (1 - 1)/2 = 0
    vol = np.array([1.0, 0, 0], dtype=np.float32).reshape(1, 1, 1, 3)
    out, idx = M.median_forward(vol)
    assert idx[0, 0, 0] == 0 and out[0, 0, 0, 0] == 0.0 and out[0, 1, 0, 0] == 1.0
    # weights that never reach 0.5 leave (0, 0) and index -1
    vol = np.full((1, 1, 1, 4), 0.1, dtype=np.float32)
    out, idx = M.median_forward(vol)
    assert idx[0, 0, 0] == -1 and out[0, 0, 0, 0] == 0 and out[0, 1, 0, 0] == 0
    # gradient: before the crossing -g0/(2 pmid), after +g0/(2 pmid), at it g0*alpha/(-pmid) + g1
    vol = np.array([0.3, 0.4, 0.3], dtype=np.float32).reshape(1, 1, 1, 3)
    grad = np.array([2.0, 5.0], dtype=np.float32).reshape(1, 2, 1, 1)
    g = M.median_backward(vol, grad)[0, 0, 0]
    alpha = (1 - 0.6 - 0.4) / 0.8
    assert np.allclose(g, [-2.0 / 0.8, 2.0 * alpha / -0.4 + 5.0, 2.0 / 0.8], atol=1e-5)


def test_oracle_gradient_sign_structure():
    """The reference's gradient is not the plain derivative of c + alpha (it is half of it before the crossing and
    mixes in the sum-to-one constraint at the crossing); what it guarantees is the structure: one negative constant
    before the crossing bin, the same constant positive after it."""
    vol, _ = make_median_volume(1, 6, 7, 21, seed=3)
    grad = np.zeros((1, 2, 6, 7), dtype=np.float32)
    grad[:, 0] = 1.0
    out, idx = M.median_forward(vol.numpy())
    g = M.median_backward(vol.numpy(), grad)
    for h in range(6):
        for w in range(7):
            c = int(idx[0, h, w])
            pm = vol[0, h, w, c].item()
            assert np.allclose(g[0, h, w, :c], -1.0 / (2 * pm), rtol=1e-6)
            assert np.allclose(g[0, h, w, c + 1:], 1.0 / (2 * pm), rtol=1e-6)


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden file not generated yet")
def test_oracle_reproduces_reference_kernel_outputs():
    z = np.load(GOLDEN)
    for i in range(int(z["n_cases"])):
        vol, grad = z[f"case{i}_vol"], z[f"case{i}_grad"]
        out, idx = M.median_forward(vol)
        g = M.median_backward(vol, grad)
        # position c + alpha: same integer part exactly, fraction to fp32 rounding
        assert np.array_equal(np.floor(out[:, 0] + 0.5), np.floor(z[f"case{i}_out"][:, 0] + 0.5))
        assert_close(torch.from_numpy(out), torch.from_numpy(z[f"case{i}_out"]), f"case {i} out", tol=1e-6)
        assert_close(torch.from_numpy(g), torch.from_numpy(z[f"case{i}_gvol"]), f"case {i} gvol", tol=1e-6)


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("case", [(1, 1, 1, 1), (1, 3, 5, 7), (2, 17, 33, 49), (1, 96, 320, 49), (3, 8, 9, 64), (1, 5, 5, 300)],
                         ids=lambda c: "n%d_%dx%d_k%d" % c)
def test_cuda_matches_oracle_bit_exact_index(case):
    from customnetworklayers_b200 import median_cuda_ext as ext
    n, h, w, k = case
    vol, grad = make_median_volume(n, h, w, k, seed=5 + k)
    if n * h * w > 4:
        vol[0, 0, 0] = 0.1 / k          # a pixel whose weights never reach 0.5
    out, idx = ext.forward_with_index(vol.cuda())
    g = ext.backward(grad.cuda(), vol.cuda())[0]
    o_ref, i_ref = M.median_forward(vol.numpy())
    g_ref = M.median_backward(vol.numpy(), grad.numpy())
    assert np.array_equal(idx.cpu().numpy(), i_ref), "crossing index must be bit-exact"
    assert np.array_equal(out.cpu().numpy(), o_ref), "position and crossing weight must be bit-exact"
    assert np.array_equal(g.cpu().numpy(), g_ref), "gradient must be bit-exact"


@pytest.mark.gpu
@pytest.mark.parametrize("k", [7, 49, 64])
def test_rows_with_negative_weights_take_the_general_scan(k):
    """Rows without negative weights are scanned by a shorter route (their running sum never falls); a negative weight
    anywhere in a row must send that row through the general rule, where the sum can cross 0.5 more than once."""
    from customnetworklayers_b200 import median_cuda_ext as ext
    vol, grad = make_median_volume(2, 9, 37, k, seed=90 + k)
    vol = vol.clone()
    vol[0, :, ::3, 1::5] *= -0.7                   # some rows only; the others stay on the short route
    vol[1, 2, 3, :] = 0.0
    vol[1, 2, 3, 0], vol[1, 2, 3, 1], vol[1, 2, 3, 2] = 0.6, -0.3, 0.4      # crosses, falls back, crosses again
    out, idx = ext.forward_with_index(vol.cuda())
    g = ext.backward(grad.cuda(), vol.cuda())[0]
    o_ref, i_ref = M.median_forward(vol.numpy())
    g_ref = M.median_backward(vol.numpy(), grad.numpy())
    assert int(i_ref[1, 2, 3]) == 0
    assert np.array_equal(idx.cpu().numpy(), i_ref), "crossing index must be bit-exact"
    assert np.array_equal(out.cpu().numpy(), o_ref), "position and crossing weight must be bit-exact"
    assert np.array_equal(g.cpu().numpy(), g_ref), "gradient must be bit-exact"


@pytest.mark.gpu
def test_cuda_matches_reference_kernels_live():
    from oracle import ref_cuda
    if not ref_cuda.median_available():
        pytest.skip("oracle/_ref/libmedianref.so not built")
    from customnetworklayers_b200 import median_cuda_ext as ext
    for (h, w, k, seed) in [(16, 24, 49, 1), (40, 56, 9, 2), (7, 5, 121, 3)]:
        vol, grad = make_median_volume(1, h, w, k, seed=seed)
        v, gr = vol.cuda(), grad.cuda()
        mine, ref = ext.forward(v)[0], ref_cuda.median_forward(v)
        # crossing weight (a copied input value) identical => same crossing bin; position to fp32 rounding (the two
        # builds contract the double-precision alpha expression differently)
        assert torch.equal(mine[:, 1], ref[:, 1])
        assert torch.equal(torch.floor(mine[:, 0] + 0.5), torch.floor(ref[:, 0] + 0.5))
        assert_close(mine, ref.cpu(), "position", tol=1e-6)
        assert_close(ext.backward(gr, v)[0], ref_cuda.median_backward(v, gr).cpu(), "gradient", tol=1e-6)


@pytest.mark.gpu
def test_median_layer_api():
    from customnetworklayers_b200.median import Median
    vol, _ = make_median_volume(1, 12, 10, 49, seed=9)
    t = vol[0].cuda().requires_grad_(True)
    pos = Median("cuda")(t)
    assert pos.shape == (12, 10)
    pos.sum().backward()
    assert t.grad.shape == t.shape and torch.isfinite(t.grad).all()
    o_ref, _ = M.median_forward(vol.numpy())
    assert np.array_equal(pos.detach().cpu().numpy(), o_ref[0, 0])
