"""Learnable weighted-median filter: oracle self-checks on CPU, GPU parity (selected tap bit-exact) through the C ABI."""
import numpy as np
import pytest
import torch

from customnetworklayers_b200.synthetic import make_median_filter_inputs
from oracle import median_ref as M
from oracle import wmedian_ref as W
from tests.parity import assert_close


def test_uniform_weights_give_the_plain_median():
    flow, _, _ = make_median_filter_inputs(1, 2, 9, 11, seed=1)
    for k in (3, 5, 7):
        p = np.full(k * k, 1.0 / (k * k), np.float32)
        out, tap, _ = W.wmedian_forward(flow.numpy(), p, k)
        win, _, _ = W._windows(flow.numpy(), k)
        assert np.array_equal(out, np.sort(win, axis=-1)[..., (k * k) // 2])


def test_selection_equals_the_reference_rule_on_the_materialised_volume():
    """Permuting the weights by the sort and running the reference layer's oracle gives the same crossing rank."""
    flow, wts, _ = make_median_filter_inputs(1, 1, 6, 7, seed=2)
    p = (wts / wts.sum()).numpy()
    out, tap, aux = W.wmedian_forward(flow.numpy(), p, 7)
    vol = p[aux["order"]][0]                      # [C=1,H,W,K] -> treat C as batch
    _, idx = M.median_forward(vol)
    assert np.array_equal(idx, aux["rank"][0])


def test_weight_gradient_sums_reference_dp_through_the_permutation():
    flow, wts, grad = make_median_filter_inputs(1, 1, 5, 6, seed=3)
    p = (wts / wts.sum()).numpy()
    _, _, aux = W.wmedian_forward(flow.numpy(), p, 7)
    g_flow, g_p = W.wmedian_backward(flow.numpy(), p, grad.numpy(), 7)
    vol = p[aux["order"]][0]
    g2 = np.zeros((1, 2, 5, 6), np.float32); g2[0, 0] = grad.numpy()[0, 0]
    dvol = M.median_backward(vol, g2)              # reference d/dp in sorted order
    ref = np.zeros(49)
    np.add.at(ref, aux["order"][0].reshape(-1), dvol.astype(np.float64).reshape(-1))
    assert np.allclose(g_p, ref, rtol=1e-6, atol=1e-6)
    assert abs(float(g_flow.sum()) - float(grad.sum())) < 1e-3       # pass-through conserves the gradient mass


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(1, 1, 1, 1, 7), (1, 2, 9, 11, 3), (2, 2, 17, 33, 5), (1, 2, 40, 56, 7), (3, 1, 8, 64, 7),
                                  (1, 1, 37, 200, 7), (2, 1, 5, 97, 5), (1, 1, 3, 70, 3)],
                         ids=lambda c: "n%d_c%d_%dx%d_k%d" % c)
def test_cuda_matches_oracle(case):
    from customnetworklayers_b200 import wmedian as wm
    n, c, h, w, k = case
    flow, wts, grad = make_median_filter_inputs(n, c, h, w, k=k, seed=10 + k)
    if h * w > 4:
        flow[0, 0, 1, :3] = 5.0                    # ties: the stable order decides
    if w >= 64:                                    # ties that enter and leave the sliding window, also across rows
        flow[0, 0, h // 2, 20:60] = -1.25
        flow[0, 0, :, 33] = flow[0, 0, :, 34]
        flow[0, 0, min(h - 1, 2), 40:50] = flow[0, 0, 0, 40:50]
    p = (wts / wts.sum()).float()
    out, tap, alpha = wm.forward(flow.cuda(), p.cuda(), k)
    g_flow, g_p = wm.backward(flow.cuda(), p.cuda(), tap, alpha, grad.cuda(), k)
    o_ref, t_ref, _ = W.wmedian_forward(flow.numpy(), p.numpy(), k)
    gf_ref, gp_ref = W.wmedian_backward(flow.numpy(), p.numpy(), grad.numpy(), k)
    assert np.array_equal(tap.cpu().numpy(), t_ref), "selected tap must be bit-exact"
    assert np.array_equal(out.cpu().numpy(), o_ref)
    assert_close(g_flow, torch.from_numpy(gf_ref), "g_flow", tol=1e-5)
    assert_close(g_p, torch.from_numpy(gp_ref), "g_weights")


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(1, 1, 20, 45, 3), (1, 2, 33, 130, 5), (2, 1, 70, 300, 7), (4, 2, 370, 1270, 7), (16, 2, 370, 1270, 7)],
                         ids=lambda c: "n%d_c%d_%dx%d_k%d" % c)
def test_sliding_kernels_give_the_bits_of_the_per_pixel_kernels(case, monkeypatch):
    """The sliding-window kernels (runs of 16, 32 or 64 pixels per thread, chosen by the size of the input; the heights
    here leave a ragged last run) against the one-thread-per-pixel kernels, which the small cases pin to the oracle."""
    from customnetworklayers_b200 import wmedian as wm
    n, c, h, w, k = case
    flow, wts, grad = make_median_filter_inputs(n, c, h, w, k=k, seed=77 + k)
    flow[0, 0, h // 2, 5:40] = 0.5                 # ties entering and leaving the window
    flow[0, 0, 3:18, w // 2] = 0.5
    flow[0, 0, :, w - 3] = flow[0, 0, :, w - 2]
    flow[0, 0, h - 3, :] = flow[0, 0, h - 2, :]
    flow, grad = flow.cuda(), grad.cuda()
    p = (wts / wts.sum()).float().cuda()
    res = {}
    for mode in ("0", "1"):
        monkeypatch.setenv("CNL_WMEDIAN_NO_SLIDE", mode)
        out, tap, alpha = wm.forward(flow, p, k)
        g_flow, g_p = wm.backward(flow, p, tap, alpha, grad, k)
        torch.cuda.synchronize()
        res[mode] = (out, tap, alpha, g_flow, g_p)
    for name, a, b in zip(("out", "tap", "alpha", "g_flow"), res["0"], res["1"]):
        assert torch.equal(a, b), name
    assert_close(res["0"][4], res["1"][4], "g_weights")


@pytest.mark.gpu
@pytest.mark.parametrize("k", [3, 7])
def test_negative_weights_cross_where_the_oracle_crosses(k):
    """With a negative weight the running sum can fall back below 0.5 and cross again; the first crossing counts.  (The
    sliding kernel scans weights that are all >= 0 by a shorter route, so this case has a path of its own.)"""
    from customnetworklayers_b200 import wmedian as wm
    flow, wts, grad = make_median_filter_inputs(1, 2, 24, 80, k=k, seed=321 + k)
    wts = wts.clone()
    wts[1::4] *= -0.6
    p = (wts / wts.sum()).float()
    assert float(p.min()) < 0
    out, tap, alpha = wm.forward(flow.cuda(), p.cuda(), k)
    g_flow, g_p = wm.backward(flow.cuda(), p.cuda(), tap, alpha, grad.cuda(), k)
    o_ref, t_ref, _ = W.wmedian_forward(flow.numpy(), p.numpy(), k)
    gf_ref, gp_ref = W.wmedian_backward(flow.numpy(), p.numpy(), grad.numpy(), k)
    assert np.array_equal(tap.cpu().numpy(), t_ref), "selected tap must be bit-exact"
    assert np.array_equal(out.cpu().numpy(), o_ref)
    assert_close(g_flow, torch.from_numpy(gf_ref), "g_flow", tol=1e-5)
    assert_close(g_p, torch.from_numpy(gp_ref), "g_weights")


@pytest.mark.gpu
def test_filter_module_learns_through_normalisation():
    from customnetworklayers_b200.wmedian import WeightedMedianFilter
    flow, wts, grad = make_median_filter_inputs(2, 2, 24, 32, seed=5)
    m = WeightedMedianFilter(7).cuda()
    with torch.no_grad():
        m.weight.copy_(wts)
    x = flow.cuda().requires_grad_(True)
    y = m(x)
    y.backward(grad.cuda())
    m.allreduce_parameter_grads()
    p = (wts / wts.sum()).float()
    _, gp_ref = W.wmedian_backward(flow.numpy(), p.numpy(), grad.numpy(), 7)
    # chain rule through p = w / sum(w)
    s = float(wts.sum())
    gp = torch.from_numpy(gp_ref)
    ref_w = (gp - (gp * p.double()).sum()) / s
    assert_close(m.weight.grad, ref_w, "weight gradient", tol=2e-4)
    assert x.grad.shape == x.shape
    # twice: deterministic
    m.weight.grad = None
    x2 = flow.cuda().requires_grad_(True)
    m(x2).backward(grad.cuda())
    assert torch.equal(x2.grad, x.grad)


@pytest.mark.gpu
def test_full_size_properties():
    """Size-independent properties at the benchmark's full size (batch 32, 2x384x1280, 7x7): the output is the window
    value at the reported tap, the pass-through gradient conserves mass, two runs give the same bits."""
    from customnetworklayers_b200 import wmedian as wm
    n, c, h, w, k = 32, 2, 384, 1280, 7
    flow, wts, grad = make_median_filter_inputs(n, c, h, w, k=k, seed=1238)
    flow, grad = flow.cuda(), grad.cuda()
    p = (wts / wts.sum()).float().cuda()
    out, tap, alpha = wm.forward(flow, p, k)
    g_flow, g_p = wm.backward(flow, p, tap, alpha, grad, k)
    out2, tap2, alpha2 = wm.forward(flow, p, k)
    g_flow2, g_p2 = wm.backward(flow, p, tap2, alpha2, grad, k)
    torch.cuda.synchronize()
    assert torch.equal(out, out2) and torch.equal(tap, tap2) and torch.equal(g_flow, g_flow2) and torch.equal(g_p, g_p2)
    assert int((tap < 0).sum()) == 0 and int(tap.max()) < k * k          # normalised weights always cross 0.5
    hh = torch.arange(h, device="cuda").view(1, 1, h, 1)
    ww = torch.arange(w, device="cuda").view(1, 1, 1, w)
    th = (hh + torch.div(tap, k, rounding_mode="floor") - k // 2).clamp(0, h - 1)
    tw = (ww + tap % k - k // 2).clamp(0, w - 1)
    picked = flow.reshape(n * c, h * w).gather(1, (th * w + tw).reshape(n * c, h * w).long()).view_as(flow)
    assert torch.equal(out, picked), "the output must be the window value at the selected tap"
    assert abs(float(g_flow.double().sum()) - float(grad.double().sum())) < 1e-2 * max(1.0, float(grad.double().abs().sum()) ** 0.5)
    assert bool(torch.isfinite(g_p).all())
