"""Differentiable quadratic fit: oracle pins (finite differences of the fit, golden vectors from the reference's own
kernels) and GPU parity through the C ABI.  The rounded integer location must be bit-exact."""
import os

import numpy as np
import pytest
import torch

from customnetworklayers_b200.synthetic import make_cost_patches, make_quadfit_inputs
from oracle import quadfit_ref as Q
from tests.parity import assert_close

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quadfit_reference_cuda.npz")


def test_fit_recovers_subpixel_maximum_of_a_parabola():
    # score(d) = -(d - 0.3)^2 sampled at -1, 0, 1 along x; flat along y
    c = lambda d: np.float32(-(d - 0.3) ** 2)
    cost5 = np.array([c(0), c(1), c(0), c(-1), c(0)], dtype=np.float32).reshape(1, 5, 1, 1)
    out = Q.quadfit_from_cost_forward(cost5)
    assert abs(out[0, 0, 0, 0] - 0.3) < 1e-6 and out[0, 1, 0, 0] == 0.0
    assert abs(out[0, 2, 0, 0] - 0.0) < 1e-6          # fitted peak value of the parabola
    # a convex stencil (a minimum) is invalid: zero offset, score = centre value
    out = Q.quadfit_from_cost_forward(-cost5)
    assert out[0, 0, 0, 0] == 0.0 and abs(out[0, 2, 0, 0] + c(0)) < 1e-7


def test_cost_gradient_matches_finite_differences():
    cost5, _ = make_cost_patches(1, 4, 5, seed=3)
    cost5 = cost5.numpy()
    grad = np.random.RandomState(1).randn(1, 3, 4, 5).astype(np.float32)
    g = Q.quadfit_from_cost_backward(cost5, grad)
    eps = 1e-3
    for k in range(5):
        for (h, w) in [(0, 0), (2, 3), (3, 4)]:
            e = np.zeros_like(cost5); e[0, k, h, w] = eps
            fp = Q.quadfit_from_cost_forward(cost5 + e).astype(np.float64)
            fm = Q.quadfit_from_cost_forward(cost5 - e).astype(np.float64)
            num = ((fp - fm)[0, :, h, w] / (2 * eps) * grad[0, :, h, w]).sum()
            assert abs(num - g[0, k, h, w]) < 2e-2 * max(1.0, abs(num)), (k, h, w, num, g[0, k, h, w])


def test_feature_gradients_match_finite_differences_where_the_location_is_stable():
    f0, f1, flow, grad = (t.numpy() for t in make_quadfit_inputs(1, 3, 8, 9, seed=4))
    g0, g1 = Q.quadfit_backward(f0, f1, flow, grad)
    loss = lambda a, b: float((Q.quadfit_forward(a, b, flow)[0].astype(np.float64) * grad).sum())
    eps = 1e-3
    rng = np.random.RandomState(0)
    for _ in range(6):
        idx = (0, rng.randint(3), rng.randint(8), rng.randint(9))
        for arr, g, which in ((f0, g0, 0), (f1, g1, 1)):
            e = np.zeros_like(arr); e[idx] = eps
            num = (loss(f0 + e, f1) - loss(f0 - e, f1)) / (2 * eps) if which == 0 else (loss(f0, f1 + e) - loss(f0, f1 - e)) / (2 * eps)
            assert abs(num - g[idx]) < 5e-2 * max(1.0, abs(num)), (which, idx, num, g[idx])


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden file not generated yet")
def test_oracle_reproduces_reference_kernel_outputs():
    z = np.load(GOLDEN)
    for i in range(int(z["n_cases"])):
        f0, f1, flow, grad = (z[f"case{i}_{k}"] for k in ("feat0", "feat1", "flow", "grad"))
        out, _, _, inside = Q.quadfit_forward(f0, f1, flow)
        g0, g1 = Q.quadfit_backward(f0, f1, flow, grad)
        assert np.array_equal(out[:, 0] != 0, z[f"case{i}_out"][:, 0] != 0)        # same validity decisions
        assert_close(torch.from_numpy(out), torch.from_numpy(z[f"case{i}_out"]), f"case {i} out")
        assert_close(torch.from_numpy(g0), torch.from_numpy(z[f"case{i}_g0"]), f"case {i} g_feat0")
        assert_close(torch.from_numpy(g1), torch.from_numpy(z[f"case{i}_g1"]), f"case {i} g_feat1")


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("case", [(1, 1, 1, 1), (1, 4, 12, 16), (2, 7, 33, 17), (1, 32, 96, 320), (3, 5, 8, 8)],
                         ids=lambda c: "n%d_c%d_%dx%d" % c)
def test_cuda_matches_oracle(case):
    from customnetworklayers_b200 import QuadFit_cuda_ext as ext
    n, c, h, w = case
    f0, f1, flow, grad = make_quadfit_inputs(n, c, h, w, seed=11 + c)
    D = [t.cuda() for t in (f0, f1, flow, grad)]
    out, loc = ext.forward_with_location(D[0], D[1], D[2])
    g0, g1 = ext.backward(D[3], D[0], D[1], D[2])
    o_ref, ix, iy, inside = Q.quadfit_forward(f0.numpy(), f1.numpy(), flow.numpy())
    r0, r1 = Q.quadfit_backward(f0.numpy(), f1.numpy(), flow.numpy(), grad.numpy())
    loc = loc.cpu().numpy()
    assert np.array_equal(loc[:, 0], np.where(inside, ix, -1)) and np.array_equal(loc[:, 1], np.where(inside, iy, -1)), \
        "rounded integer location must be bit-exact"
    assert_close(out, torch.from_numpy(o_ref), "out")
    assert_close(g0, torch.from_numpy(r0), "g_feat0")
    assert_close(g1, torch.from_numpy(r1), "g_feat1")


@pytest.mark.gpu
def test_rounding_of_half_integer_locations_follows_the_double_path():
    """floor(idx + 0.5) is evaluated in double on the fp32 sum w + flow; values just below .5 must round down."""
    from customnetworklayers_b200 import QuadFit_cuda_ext as ext
    h, w, c = 4, 64, 2
    f0 = torch.randn(1, c, h, w); f1 = torch.randn(1, c, h, w)
    flow = torch.zeros(1, 2, h, w)
    flow[0, 0] = torch.tensor(np.nextafter(np.float32(0.5), np.float32(0.0)))     # largest float below 0.5
    flow[0, 0, 1] = 0.5
    flow[0, 0, 2] = 1.4999999
    _, loc = ext.forward_with_location(f0.cuda(), f1.cuda(), flow.cuda())
    _, ix, iy, inside = Q.quadfit_forward(f0.numpy(), f1.numpy(), flow.numpy())
    assert np.array_equal(loc.cpu().numpy()[0, 0], np.where(inside[0], ix[0], -1))


@pytest.mark.gpu
def test_cost_variant_and_layers():
    from customnetworklayers_b200 import QuadFit_cuda_ext as ext
    from customnetworklayers_b200.QuadFitting import QuadFittingFromCost, QuadFittingFromFlow
    cost5, off = make_cost_patches(2, 20, 28, seed=5)
    grad = torch.randn(2, 3, 20, 28)
    out = ext.cost_forward(cost5.cuda())
    g = ext.cost_backward(grad.cuda(), cost5.cuda())
    assert_close(out, torch.from_numpy(Q.quadfit_from_cost_forward(cost5.numpy())), "cost out")
    assert_close(g, torch.from_numpy(Q.quadfit_from_cost_backward(cost5.numpy(), grad.numpy())), "cost grad")
    # the fit lands near the true sub-pixel offsets (noise 0.05 on a bowl of curvature >= 0.5)
    assert float((out[:, :2].cpu() - off).abs().mean()) < 0.12
    t = cost5.cuda().requires_grad_(True)
    QuadFittingFromCost()(t).sum().backward()
    assert t.grad.shape == t.shape
    # HWC layer with a 3-channel flow, as the reference's layer asserts
    f0, f1, flow, grad3 = make_quadfit_inputs(1, 6, 16, 24, seed=8)
    hwc = lambda x: x[0].permute(1, 2, 0).contiguous().cuda()
    flow3 = torch.cat([flow, torch.zeros(1, 1, 16, 24)], dim=1)
    a, b = hwc(f0).requires_grad_(True), hwc(f1).requires_grad_(True)
    sol = QuadFittingFromFlow("cuda")(a, b, hwc(flow3))
    assert sol.shape == (16, 24, 3)
    o_ref, *_ = Q.quadfit_forward(f0.numpy(), f1.numpy(), flow.numpy())
    assert_close(sol.permute(2, 0, 1).unsqueeze(0), torch.from_numpy(o_ref), "layer out")
    sol.backward(hwc(grad3))
    assert a.grad is not None and b.grad is not None


@pytest.mark.gpu
def test_cuda_matches_reference_kernels_live():
    from oracle import ref_cuda
    if not ref_cuda.quadfit_available():
        pytest.skip("oracle/_ref/libquadfitref.so not built")
    from customnetworklayers_b200 import QuadFit_cuda_ext as ext
    for (n, c, h, w, seed) in [(1, 8, 24, 40, 1), (2, 3, 17, 13, 2)]:
        f0, f1, flow, grad = (t.cuda() for t in make_quadfit_inputs(n, c, h, w, seed=seed))
        ref_out = ref_cuda.quadfit_forward(f0, f1, flow)
        ref_g0, ref_g1 = ref_cuda.quadfit_backward(f0, f1, flow, grad)
        out = ext.forward(f0, f1, flow)[0]
        g0, g1 = ext.backward(grad, f0, f1, flow)
        assert torch.equal(out[:, 0] != 0, ref_out[:, 0] != 0)
        assert_close(out, ref_out.cpu(), "out")
        assert_close(g0, ref_g0.cpu(), "g_feat0")
        assert_close(g1, ref_g1.cpu(), "g_feat1")
