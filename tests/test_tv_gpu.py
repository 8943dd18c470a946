"""Parity of the CUDA TV-FISTA layer with the float64 CPU oracle, through the C ABI.

Tolerance: 1e-4 relative, norm-wise (max-norm and L2) per output tensor.  The forward pass and the stored
iterate history are compared end to end.  The reverse sweep is discontinuous in the iterates at the Huber
thresholds, so it is compared with the oracle's reverse sweep run on exactly the iterates the device stored;
the end-to-end gradient difference is reported next to the oracle's own fp32-vs-fp64 difference."""
import pytest
import torch

from oracle import tv_ref as R
from tests.parity import REL_TOL, assert_close, rel_errors

pytestmark = pytest.mark.gpu

GRAD_NAMES = ["g_wx", "g_wy", "g_c", "g_b", "g_init"]


@pytest.fixture(scope="module")
def ext():
    from customnetworklayers_b200 import tvInpaint_cuda_ext
    from customnetworklayers_b200 import _lib
    _lib.load()
    return tvInpaint_cuda_ext


def _dev(I):
    return {k: v.cuda() for k, v in I.items()}


def _run_cuda(ext, D, its, pid):
    sol = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)[0]
    hist, cky = ext.read_history(pid, D["b"], its)
    grads = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)
    torch.cuda.synchronize()
    return sol, hist, cky, grads


CASES = [
    # n, ch, h, w, its
    (1, 1, 1, 1, 2),
    (1, 2, 1, 37, 4),
    (1, 2, 29, 1, 4),
    (1, 1, 17, 33, 20),
    (1, 3, 17, 33, 21),
    (2, 2, 40, 72, 20),
    (1, 2, 96, 320, 20),      # the CPU-runnable configuration
    (1, 2, 33, 65, 50),
    (1, 2, 64, 96, 100),
    (3, 2, 50, 70, 9),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "n%d_c%d_%dx%d_its%d" % c)
def test_forward_and_history_match_oracle(ext, case):
    n, ch, h, w, its = case
    I = R.make_inputs(n, ch, h, w, seed=1234 + h + w)
    D = _dev(I)
    ext.set_option(2, 1, 0)
    sol, hist, cky, _ = _run_cuda(ext, D, its, 2)
    ref_sol, ref_hist, ref_cky = R.tv_forward_history(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    assert_close(sol, ref_sol, "solution")
    assert_close(hist, ref_hist, "history")
    assert_close(cky, ref_cky, "checkpointed y")


@pytest.mark.parametrize("case", CASES, ids=lambda c: "n%d_c%d_%dx%d_its%d" % c)
def test_reverse_sweep_matches_oracle_on_device_history(ext, case):
    n, ch, h, w, its = case
    I = R.make_inputs(n, ch, h, w, seed=4321 + h + w)
    D = _dev(I)
    ext.release(3)
    ext.set_option(3, 1, 0)          # conditioner off: pure reverse sweep + sanitiser + scalings
    sol, hist, cky, grads = _run_cuda(ext, D, its, 3)
    ref = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, None, hist=hist.cpu(), ckpt_y=cky.cpu())
    for name, g, r in zip(GRAD_NAMES, grads, ref):
        assert_close(g, r, name)


FUSE_CASES = [(2, 2, 40, 72, 20), (1, 3, 33, 64, 21), (1, 2, 64, 96, 100), (2, 1, 7, 8, 6), (1, 2, 100, 260, 14)]


@pytest.mark.parametrize("fuse", [1, 2, 3, 4])
@pytest.mark.parametrize("case", FUSE_CASES, ids=lambda c: "n%d_c%d_%dx%d_its%d" % c)
def test_every_fuse_factor_matches_oracle(ext, case, fuse):
    """The temporally blocked kernels (2..4 iterations per launch) and the one-launch-per-iteration kernels must all
    agree with the oracle; widths are multiples of 4 so the blocked path is the one that runs for fuse > 1."""
    n, ch, h, w, its = case
    I = R.make_inputs(n, ch, h, w, seed=777 + h + w + its)
    D = _dev(I)
    ext.release(2)
    ext.set_option(2, 1, 0)
    ext.set_option(2, 2, fuse)
    try:
        sol, hist, cky, grads = _run_cuda(ext, D, its, 2)
    finally:
        ext.set_option(2, 2, 0)
    ref_sol, ref_hist, ref_cky = R.tv_forward_history(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    assert_close(sol, ref_sol, "solution")
    assert_close(hist, ref_hist, "history")
    assert_close(cky, ref_cky, "checkpointed y")
    ref = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, None, hist=hist.cpu(), ckpt_y=cky.cpu())
    for name, g, r in zip(GRAD_NAMES, grads, ref):
        assert_close(g, r, name)


def test_end_to_end_gradient_gap_is_reported_and_bounded(ext):
    """End to end (oracle recomputes its own fp64 forward) the difference is dominated by threshold flips; it must
    stay within a small multiple of what the fp32 oracle itself shows against the fp64 oracle."""
    n, ch, h, w, its = 1, 2, 96, 320, 20
    I = R.make_inputs(n, ch, h, w, seed=1234)
    D = _dev(I)
    ext.release(4)
    ext.set_option(4, 1, 0)
    _, _, _, grads = _run_cuda(ext, D, its, 4)
    _, ck64 = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its, torch.float64)
    g64 = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck64, torch.float64)
    _, ck32 = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its, torch.float32)
    g32 = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck32, torch.float32)
    for name, g, r64, r32 in zip(GRAD_NAMES, grads, g64, g32):
        e = rel_errors(g, r64)
        e32 = rel_errors(r32, r64)
        print(f"{name}: cuda-vs-fp64 max {e[0]:.2e} l2 {e[1]:.2e} | oracle fp32-vs-fp64 max {e32[0]:.2e} l2 {e32[1]:.2e}")
        assert e[1] <= max(REL_TOL, 5.0 * e32[1]), name


def test_batch_equals_single_calls_bit_for_bit(ext):
    n, ch, h, w, its = 3, 2, 45, 67, 12
    I = R.make_inputs(n, ch, h, w, seed=99)
    D = _dev(I)
    for pid in (5, 6):
        ext.release(pid)
        ext.set_option(pid, 1, 0)
    sol, _, _, grads = _run_cuda(ext, D, its, 5)
    for i in range(n):
        Di = {k: v[i:i + 1].contiguous() for k, v in D.items()}
        s1, _, _, g1 = _run_cuda(ext, Di, its, 6)
        assert torch.equal(s1[0], sol[i])
        for name, a, b in zip(GRAD_NAMES, g1, grads):
            assert torch.equal(a[0], b[i]), name


def test_python_layer_autograd_and_hwc_convention(ext):
    from customnetworklayers_b200 import TVInpaint
    h, w, ch, its = 24, 40, 2, 10
    I = R.make_inputs(1, ch, h, w, seed=5)
    hwc = lambda t: t[0].permute(1, 2, 0).contiguous().cuda()
    leaves = [hwc(I[k]).requires_grad_(True) for k in ("wx", "wy", "c", "b", "init")]
    layer = TVInpaint("cuda", its, pid=7)
    ext.release(7)
    out = layer(*leaves)
    assert out.shape == (h, w, ch)
    out.backward(hwc(I["grad"]))
    ref_sol, hist, cky = R.tv_forward_history(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
    assert_close(out.permute(2, 0, 1).unsqueeze(0), ref_sol, "layer output")
    for t in leaves:
        assert t.grad is not None and t.grad.shape == t.shape and torch.isfinite(t.grad).all()
    # batched extension: N x H x W x C
    I3 = R.make_inputs(3, ch, h, w, seed=6)
    nhwc = lambda t: t.permute(0, 2, 3, 1).contiguous().cuda()
    out3 = layer(*[nhwc(I3[k]) for k in ("wx", "wy", "c", "b", "init")])
    ref3, _ = R.tv_forward_raw(I3["wx"], I3["wy"], I3["c"], I3["b"], I3["init"], its)
    assert_close(out3.permute(0, 3, 1, 2), ref3, "batched layer output")


def test_stale_history_and_wrong_shapes_are_refused(ext):
    """A slot keeps its last forward pass only: the backward pass of an earlier forward on the same id must raise,
    not return gradients of the other problem; wrongly shaped weight maps are refused before any kernel runs."""
    from customnetworklayers_b200 import TVInpaintingFunction
    I = R.make_inputs(1, 2, 16, 24, seed=3)
    D = _dev(I)
    ext.release(7)
    first = [D[k].clone().requires_grad_(True) for k in ("wx", "wy", "c", "b", "init")]
    second = [D[k].clone().requires_grad_(True) for k in ("wx", "wy", "c", "b", "init")]
    out1 = TVInpaintingFunction.apply(*first, 6, 7)
    out2 = TVInpaintingFunction.apply(*second, 6, 7)
    with pytest.raises(RuntimeError, match="replaced the history"):
        out1.backward(D["grad"])
    out2.backward(D["grad"])
    assert all(t.grad is not None for t in second)
    ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 6, 7)
    with pytest.raises(RuntimeError, match=r"d_c must have shape \[N,1,H,W\]"):
        ext.backward(D["grad"], D["wx"], D["wy"], D["c"][:, :, :8].contiguous(), D["b"], 6, 7)
    with pytest.raises(RuntimeError, match=r"d_x must have shape \[N,1,H,W\]"):
        ext.backward(D["grad"], D["b"], D["wy"], D["c"], D["b"], 6, 7)
    ext.release(7)


def test_properties(ext):
    n, ch, h, w, its = 1, 2, 32, 48, 30
    I = R.make_inputs(n, ch, h, w, seed=8)
    D = _dev(I)
    # zero edge weights decouple the pixels: with c = 0 nothing moves at all
    z = torch.zeros_like(D["wx"])
    out = ext.forward(z, z, torch.zeros_like(D["c"]), D["b"], D["init"], its, 8)[0]
    assert torch.equal(out, D["init"])
    # huge confidence pins the solution to b wherever |x05 - b| <= 1 + c
    big = torch.full_like(D["c"], 1e6)
    out = ext.forward(z, z, big, D["b"], D["b"] + 0.5, its, 8)[0]
    assert float((out - D["b"]).abs().max()) < 1e-3
    # a constant image is a fixed point of the smoothing step when c = 0
    const = torch.full_like(D["b"], 3.25)
    out = ext.forward(D["wx"], D["wy"], torch.zeros_like(D["c"]), D["b"], const, its, 8)[0]
    assert torch.equal(out, const)
    # run twice: deterministic
    a = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 8)[0]
    ga = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 8)
    b2 = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 8)[0]
    gb = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 8)
    assert torch.equal(a, b2) and all(torch.equal(x, y) for x, y in zip(ga, gb))
    # inputs are not modified
    assert torch.equal(D["wx"].cpu(), I["wx"]) and torch.equal(D["c"].cpu(), I["c"])


def test_nonfinite_upstream_gradient_is_zeroed(ext):
    n, ch, h, w, its = 1, 2, 20, 24, 8
    I = R.make_inputs(n, ch, h, w, seed=10)
    D = _dev(I)
    ext.release(9)
    ext.set_option(9, 1, 0)
    g = D["grad"].clone()
    g[0, 0, 3, 4] = float("nan")
    g[0, 1, 7, 9] = float("inf")
    ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 9)
    hist, cky = ext.read_history(9, D["b"], its)
    grads = ext.backward(g, D["wx"], D["wy"], D["c"], D["b"], its, 9)
    ref = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], g.cpu(), its, None, hist=hist.cpu(), ckpt_y=cky.cpu())
    for name, a, r in zip(GRAD_NAMES, grads, ref):
        assert torch.isfinite(a).all()
        assert_close(a, r, name)


def test_error_codes(ext):
    I = R.make_inputs(1, 2, 8, 8, seed=1)
    D = _dev(I)
    with pytest.raises(RuntimeError, match="outside 0..9"):
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 4, 10)
    with pytest.raises(RuntimeError, match="its must be"):
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 1, 0)
    ext.release(1)
    with pytest.raises(RuntimeError, match="preceding forward"):
        ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], 4, 1)
    ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 4, 1)
    with pytest.raises(RuntimeError, match="preceding forward"):
        ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], 6, 1)       # different its


def test_conditioner_matches_oracle_state_machine(ext):
    """Twelve forward/backward rounds on one id; the 12th gets a 30x larger upstream gradient, which the running-mean
    conditioner must rescale exactly like the oracle's transcription does."""
    n, ch, h, w, its = 1, 2, 16, 24, 6
    I = R.make_inputs(n, ch, h, w, seed=12)
    D = _dev(I)
    ext.release(0)
    ext.set_option(0, 1, 1)
    st = R.IdState()
    for r in range(12):
        scale = 30.0 if r == 11 else 1.0
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 0)
        hist, cky = ext.read_history(0, D["b"], its)
        grads = ext.backward(D["grad"] * scale, D["wx"], D["wy"], D["c"], D["b"], its, 0)
        ref = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"] * scale, its, None, state=st,
                                hist=hist.cpu(), ckpt_y=cky.cpu())
        for name, a, rr in zip(GRAD_NAMES, grads, ref):
            assert_close(a, rr, f"round {r} {name}")
    # the last round was rescaled (not an identity): compare with an unconditioned run
    ext.release(1)
    ext.set_option(1, 1, 0)
    ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 1)
    plain = ext.backward(D["grad"] * 30.0, D["wx"], D["wy"], D["c"], D["b"], its, 1)
    ratio = float(grads[3].norm() / plain[3].norm())
    assert 0.2 < ratio < 0.5


def test_conditioner_kill_branch_matches_oracle_state_machine(ext):
    """After ten runs an upstream gradient 100 times larger than usual exceeds 50 times the running mean of every
    returned gradient: all five are zeroed (TVInpaintFista.cu:132-140) and the running means move as the oracle's
    transcription says, which the following ordinary rounds (one of them rescaled) show."""
    n, ch, h, w, its = 1, 2, 16, 24, 6
    I = R.make_inputs(n, ch, h, w, seed=13)
    D = _dev(I)
    ext.release(0)
    ext.set_option(0, 1, 1)
    st = R.IdState()
    scales = [1.0] * 11 + [100.0, 1.0, 30.0, 1.0]
    for r, scale in enumerate(scales):
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 0)
        hist, cky = ext.read_history(0, D["b"], its)
        grads = ext.backward(D["grad"] * scale, D["wx"], D["wy"], D["c"], D["b"], its, 0)
        ref = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"] * scale, its, None, state=st,
                                hist=hist.cpu(), ckpt_y=cky.cpu())
        for name, a, rr in zip(GRAD_NAMES, grads, ref):
            assert_close(a, rr, f"round {r} {name}")
        if scale == 100.0:
            assert all(float(rr.abs().max()) == 0.0 for rr in ref), "the oracle kills this round"
            assert all(float(a.abs().max()) == 0.0 for a in grads), "every returned gradient is zeroed"
    ext.release(0)


def test_nonfinite_returned_gradient_after_ten_runs_is_killed(ext):
    """A NaN in the data term at one pixel spreads through a patch of the iterates and into the returned gradients.
    The sanitiser zeroes such entries; after ten runs the conditioner treats a gradient that contained one as a spike
    (running mean restarted from 1000 x its value, TVInpaintFista.cu:171) and zeroes the whole tensor.  The reference's
    mean then depends on where the entry sits; here it does not, so only the outcome is checked: finite outputs, the
    affected tensors zeroed, and ordinary gradients again on the next clean run."""
    n, ch, h, w, its = 1, 2, 16, 24, 6
    I = R.make_inputs(n, ch, h, w, seed=14)
    D = _dev(I)
    ext.release(0)
    ext.set_option(0, 1, 1)
    clean = None
    for r in range(11):
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 0)
        clean = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 0)
    bad_b = D["b"].clone()
    bad_b[0, 0, 12, 17] = float("nan")
    ext.forward(D["wx"], D["wy"], D["c"], bad_b, D["init"], its, 0)
    hist, _ = ext.read_history(0, D["b"], its)
    assert not bool(torch.isfinite(hist).all()), "the iterates must contain non-finite values for this test to bite"
    grads = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], bad_b, its, 0)
    assert all(bool(torch.isfinite(g).all()) for g in grads)
    assert float(grads[2].abs().max()) == 0.0 and float(grads[3].abs().max()) == 0.0, "g_c and g_b carried NaNs: killed"
    ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 0)
    again = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 0)
    for name, a, b2 in zip(GRAD_NAMES, again, clean):
        assert torch.equal(a, b2), name + ": a clean run after the spike is an ordinary run"
    ext.release(0)


FLOW_CASES = [(2, 2, 40, 72, 20), (1, 3, 33, 64, 21), (1, 2, 100, 260, 14), (3, 1, 50, 128, 8), (1, 2, 24, 40, 2),
              (2, 2, 64, 128, 50), (1, 2, 384, 1280, 100), (5, 2, 384, 1280, 12)]


@pytest.mark.parametrize("case", FLOW_CASES, ids=lambda c: "n%d_c%d_%dx%d_its%d" % c)
def test_single_launch_sweep_gives_the_bits_of_one_launch_per_time_block(ext, case):
    """The cooperative single-launch sweeps (tiles ordered by progress counters) and the one-launch-per-time-block path
    run the same arithmetic on the same tiles, so every stored iterate, checkpoint, solution and gradient must be equal
    bit for bit; iteration counts that are and are not multiples of the time block included."""
    from customnetworklayers_b200 import _lib
    n, ch, h, w, its = case
    D = _dev(R.make_inputs(n, ch, h, w, seed=31 + h + w))
    a_id, b_id = 2, 3
    res = {}
    for pid, flow in ((a_id, 1), (b_id, 0)):
        ext.release(pid)
        ext.set_option(pid, _lib.OPT_CONDITIONER, 0)
        ext.set_option(pid, _lib.OPT_FLOW, flow)
        try:
            res[flow] = _run_cuda(ext, D, its, pid)
        finally:
            ext.set_option(pid, _lib.OPT_FLOW, 1)
            ext.set_option(pid, _lib.OPT_CONDITIONER, 1)
    for name, a, b2 in zip(("solution", "history", "checkpoints"), res[1][:3], res[0][:3]):
        assert torch.equal(a, b2), name
    for name, a, b2 in zip(GRAD_NAMES, res[1][3], res[0][3]):
        assert torch.equal(a, b2), name
    ext.release(a_id)
    ext.release(b_id)


def test_a_wait_that_cannot_end_stops_the_sweep_and_is_reported(ext):
    """Bounded waits: with progress counters that no tile can satisfy (self-test value of the option) the sweep's waits
    run out after about a second, every CTA leaves, the context stays usable and the next call reports what happened."""
    from customnetworklayers_b200 import _lib
    D = _dev(R.make_inputs(1, 2, 40, 72, seed=5))
    pid = 2
    ext.release(pid)
    ext.set_option(pid, _lib.OPT_FLOW, 2)
    try:
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 12, pid)
        torch.cuda.synchronize()                     # returns: nothing hangs
    finally:
        ext.set_option(pid, _lib.OPT_FLOW, 1)
    with pytest.raises(RuntimeError, match="gave up waiting"):
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 12, pid)
    # reported once; the library works as before afterwards
    sol = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 12, pid)[0]
    ext.set_option(3, _lib.OPT_FLOW, 0)
    ref = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], 12, 3)[0]
    ext.set_option(3, _lib.OPT_FLOW, 1)
    assert torch.equal(sol, ref)
    ext.release(pid)
    ext.release(3)


def test_lambda_gradients_on_two_streams_at_once_do_not_disturb_each_other(ext):
    """The reduction runs in one launch whose last block adds the block partials; which block is last is decided by a
    ticket word that the library hands out per call.  Many calls in flight on two streams, with inputs of different
    sizes, must each give the sum of their own inputs, the same bits every time."""
    gen = torch.Generator().manual_seed(77)
    sizes = [2 * 384 * 1280, 8 * 384 * 1280]
    a = [torch.randn(n, generator=gen).cuda() for n in sizes]
    b = [torch.rand(n, generator=gen).cuda() for n in sizes]
    exact = [float((x.double() * y.double()).sum()) for x, y in zip(a, b)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    results = [[], []]
    for _ in range(40):
        for k, st in enumerate(streams):
            with torch.cuda.stream(st):
                results[k].append(ext.lambda_grad(a[k], b[k]))
    torch.cuda.synchronize()
    for k in range(2):
        vals = torch.cat(results[k]).cpu()
        assert bool((vals == vals[0]).all()), "the same inputs must give the same bits on every call"
        assert abs(float(vals[0]) - exact[k]) <= 1e-4 * max(1.0, abs(exact[k]))


def test_host_pipeline_matches_direct_calls(ext):
    """The chunked host-buffer API (copies overlapped with kernels) must give exactly the per-image results of the
    direct device API, for chunk sizes that do and do not divide the batch."""
    from customnetworklayers_b200.host_pipeline import HostPipeline, tv_fwd_bwd_from_host
    n, ch, h, w, its = 5, 2, 40, 64, 10
    I = R.make_inputs(n, ch, h, w, seed=44)
    host = {k: v.pin_memory() for k, v in I.items()}
    like = {"sol": "b", "g_wx": "wx", "g_wy": "wy", "g_c": "c", "g_b": "b", "g_init": "b"}
    D = _dev(I)
    ext.release(5)
    ext.set_option(5, 1, 0)
    lam = torch.full((1,), 0.75, device="cuda")
    c = D["c"] * lam
    sol = ext.forward(D["wx"], D["wy"], c, D["b"], D["init"], its, 5)[0]
    grads = ext.backward(D["grad"], D["wx"], D["wy"], c, D["b"], its, 5)
    g_lam = ext.lambda_grad(grads[2], D["c"])
    torch.cuda.synchronize()
    pipe = HostPipeline("cuda:0")
    for chunk in (2, 5, 1):
        out = {k: torch.zeros_like(host[like[k]]).pin_memory() for k in like}
        hl = torch.zeros(1).pin_memory()
        tv_fwd_bwd_from_host(pipe, host, out, its, 5, lam=lam, chunk=chunk, host_lam_grad=hl)
        torch.cuda.synchronize()
        assert torch.equal(out["sol"], sol.cpu())
        for name, g in zip(("g_wx", "g_wy", "g_c", "g_b", "g_init"), grads):
            assert torch.equal(out[name], g.cpu()), (chunk, name)
        assert abs(float(hl) - float(g_lam)) <= 1e-5 * max(1.0, abs(float(g_lam)))


# Checkpoint-only storage with segment-wise recomputation in the backward pass (OPT_RECOMPUTE).
RECOMPUTE_CASES = [(1, 1, 8, 8, 2), (2, 2, 40, 72, 20), (1, 3, 24, 44, 21), (1, 2, 96, 320, 50), (2, 1, 30, 128, 100)]


@pytest.mark.parametrize("case", RECOMPUTE_CASES, ids=lambda c: "n%d_c%d_%dx%d_its%d" % c)
def test_recompute_mode_matches_full_history(ext, case):
    from customnetworklayers_b200 import _lib
    n, ch, h, w, its = case
    D = _dev(R.make_inputs(n, ch, h, w, seed=77 + h + w))
    full_id, rec_id = 4, 5
    for pid in (full_id, rec_id):
        ext.release(pid)
        ext.set_option(pid, _lib.OPT_CONDITIONER, 0)
    ext.set_option(rec_id, _lib.OPT_RECOMPUTE, 1)
    try:
        sol_f = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, full_id)[0]
        g_f = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, full_id)
        sol_r = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, rec_id)[0]
        _, cky_f = ext.read_history(full_id, D["b"], its)
        lib = _lib.load()
        k = lib.cnl_tv_num_checkpoints(rec_id)
        assert k == cky_f.shape[0]
        ck = torch.empty_like(D["b"])
        for i in range(k):      # the checkpoints are the same iterates in both modes
            _lib.check(lib.cnl_tv_read_checkpoint(rec_id, i, ck.data_ptr(), torch.cuda.current_stream().cuda_stream), "ckpt")
            assert torch.equal(ck, cky_f[i])
        g_r = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, rec_id)
        g_r2 = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, rec_id)    # rebuilds the last segment too
        torch.cuda.synchronize()
        assert torch.equal(sol_f, sol_r), "the forward pass must not depend on how launches are grouped"
        for name, a, b2, c2 in zip(GRAD_NAMES, g_f, g_r, g_r2):
            assert torch.equal(b2, c2), name + ": repeated backward differs"
            # launches are grouped differently, so the per-pixel sums are associated differently
            assert_close(b2.cpu(), a.cpu(), name, tol=1e-5)
    finally:
        ext.set_option(rec_id, _lib.OPT_RECOMPUTE, 0)
        for pid in (full_id, rec_id):
            ext.set_option(pid, _lib.OPT_CONDITIONER, 1)
            ext.release(pid)


def test_history_budget_switches_to_recomputation(ext, monkeypatch):
    from customnetworklayers_b200 import _lib
    n, ch, h, w, its = 1, 2, 96, 320, 100
    D = _dev(R.make_inputs(n, ch, h, w, seed=5))
    pid = 6
    ext.release(pid)
    ext.set_option(pid, _lib.OPT_CONDITIONER, 0)
    try:
        sol = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)[0]
        grads = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)
        torch.cuda.synchronize()
        ext.release(pid)
        # full history: 118 volumes of 245,760 B = 29 MB; checkpoints + one segment: about 10 MB
        monkeypatch.setenv("CNL_MAX_ARENA_GB", "0.015")
        sol2 = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)[0]
        with pytest.raises(RuntimeError):
            ext.read_history(pid, D["b"], its)          # iteration 0 is not resident in this mode
        grads2 = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)
        torch.cuda.synchronize()
        assert torch.equal(sol, sol2)
        for name, a, b2 in zip(GRAD_NAMES, grads, grads2):
            assert_close(b2.cpu(), a.cpu(), name, tol=1e-5)
        monkeypatch.setenv("CNL_MAX_ARENA_GB", "0.001")
        ext.release(pid)
        with pytest.raises(RuntimeError):
            ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)       # not even the checkpoints fit
    finally:
        monkeypatch.delenv("CNL_MAX_ARENA_GB", raising=False)
        ext.set_option(pid, _lib.OPT_CONDITIONER, 1)
        ext.release(pid)


def test_full_size_properties(ext):
    """Size-independent properties at the benchmark's full size (batch 8, 2x384x1280, 100 iterations), where the
    oracle would take minutes: fixed point, batch independence, linearity of the reverse sweep, storage modes."""
    from customnetworklayers_b200 import _lib
    from customnetworklayers_b200.synthetic import make_inputs
    n, ch, h, w, its = 8, 2, 384, 1280, 100
    D = _dev(make_inputs(n, ch, h, w, seed=4321))
    pid, pid1 = 7, 8
    for p in (pid, pid1):
        ext.release(p)
        ext.set_option(p, _lib.OPT_CONDITIONER, 0)
    try:
        # a constant image is a fixed point of the smoothing step when c = 0
        const = torch.full_like(D["b"], -1.75)
        out = ext.forward(D["wx"], D["wy"], torch.zeros_like(D["c"]), D["b"], const, its, pid)[0]
        assert torch.equal(out, const)
        sol = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)[0]
        g1 = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)
        assert all(bool(torch.isfinite(t).all()) for t in (sol,) + tuple(g1))
        # the reverse sweep is linear in the upstream gradient; a factor of two is exact in binary floating point
        g2 = ext.backward(2.0 * D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)
        for name, a, b2 in zip(GRAD_NAMES, g1, g2):
            assert float((2.0 * a - b2).abs().max()) <= 1e-30, name + ": backward(2 g) != 2 backward(g)"
        # images of a batch do not interact: image 5 alone gives the same bits
        k = 5
        one = {key: D[key][k:k + 1].contiguous() for key in D}
        sol_k = ext.forward(one["wx"], one["wy"], one["c"], one["b"], one["init"], its, pid1)[0]
        gk = ext.backward(one["grad"], one["wx"], one["wy"], one["c"], one["b"], its, pid1)
        assert torch.equal(sol_k[0], sol[k])
        for name, a, b2 in zip(GRAD_NAMES, g1, gk):
            assert torch.equal(a[k], b2[0]), name + ": batch member differs from the single call"
        # checkpoint-only storage gives the same solution and the same gradients up to the association of sums
        ext.release(pid1)
        ext.set_option(pid1, _lib.OPT_RECOMPUTE, 1)
        sol_r = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid1)[0]
        gr = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid1)
        torch.cuda.synchronize()
        assert torch.equal(sol_r, sol)
        for name, a, b2 in zip(GRAD_NAMES, g1, gr):
            assert_close(b2, a, name, tol=1e-5)
    finally:
        ext.set_option(pid1, _lib.OPT_RECOMPUTE, 0)
        for p in (pid, pid1):
            ext.set_option(p, _lib.OPT_CONDITIONER, 1)
            ext.release(p)


def test_widths_and_pointers_that_need_staging(ext):
    """Rows that are not a multiple of four floats (e.g. the 1242-pixel rows of a common flow benchmark) and tensors
    that are not 16-byte aligned run the same temporally blocked kernels on zero-padded copies."""
    from customnetworklayers_b200 import _lib
    pid = 9
    ext.release(pid)
    ext.set_option(pid, _lib.OPT_CONDITIONER, 0)
    try:
        n, ch, h, w, its = 2, 2, 30, 1242, 10
        I = R.make_inputs(n, ch, h, w, seed=4242)
        D = _dev(I)
        sol, hist, cky, grads = _run_cuda(ext, D, its, pid)
        ref_sol, ref_hist, ref_cky = R.tv_forward_history(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
        assert_close(sol, ref_sol, "solution")
        assert_close(hist, ref_hist, "history")
        assert_close(cky, ref_cky, "checkpoints")
        ref = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, None, hist=hist.cpu(), ckpt_y=cky.cpu())
        for name, g, r in zip(GRAD_NAMES, grads, ref):
            assert_close(g, r, name)
        # checkpoint-only storage on top of the staging
        ext.set_option(pid, _lib.OPT_RECOMPUTE, 1)
        sol_r = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)[0]
        g_r = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)
        assert torch.equal(sol_r, sol)
        for name, a, b2 in zip(GRAD_NAMES, grads, g_r):
            assert_close(b2, a, name, tol=1e-5)
        ext.set_option(pid, _lib.OPT_RECOMPUTE, 0)
        # misaligned tensors of an aligned shape give the bits of the aligned call
        n, ch, h, w, its = 1, 2, 24, 64, 12
        I = R.make_inputs(n, ch, h, w, seed=77)
        D = _dev(I)
        sol_a = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)[0]
        g_a = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)

        def shifted(t):              # same values, storage offset of one float
            buf = torch.empty(t.numel() + 1, device=t.device, dtype=t.dtype)
            view = buf[1:].view(t.shape)
            view.copy_(t)
            return view
        U = {k: shifted(v) for k, v in D.items()}
        assert all(v.data_ptr() % 16 != 0 for v in U.values())
        sol_u = ext.forward(U["wx"], U["wy"], U["c"], U["b"], U["init"], its, pid)[0]
        g_u = ext.backward(U["grad"], U["wx"], U["wy"], U["c"], U["b"], its, pid)
        torch.cuda.synchronize()
        assert torch.equal(sol_u, sol_a)
        for name, a, b2 in zip(GRAD_NAMES, g_a, g_u):
            assert torch.equal(a, b2), name
    finally:
        ext.set_option(pid, _lib.OPT_RECOMPUTE, 0)
        ext.set_option(pid, _lib.OPT_CONDITIONER, 1)
        ext.release(pid)


def _random_cases(count, seed):
    import random
    rng = random.Random(seed)
    cases = []
    for _ in range(count):
        cases.append((rng.randint(1, 3), rng.randint(1, 3), rng.randint(1, 70), rng.randint(1, 300), rng.randint(2, 15),
                      rng.random() < 0.4))
    return cases


@pytest.mark.parametrize("case", _random_cases(14, 2024), ids=lambda c: "n%d_c%d_%dx%d_its%d_rec%d" % c)
def test_random_shapes_match_oracle(ext, case):
    """Seeded random shapes (any width, hence both the in-place and the staged path; tiles that straddle the image in
    both directions; with and without checkpoint-only storage) against the oracle."""
    from customnetworklayers_b200 import _lib
    n, ch, h, w, its, rec = case
    I = R.make_inputs(n, ch, h, w, seed=h * 1000 + w)
    D = _dev(I)
    pid = 1
    ext.release(pid)
    ext.set_option(pid, _lib.OPT_CONDITIONER, 0)
    ext.set_option(pid, _lib.OPT_RECOMPUTE, 1 if rec else 0)
    try:
        sol = ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)[0]
        grads = ext.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, pid)
        torch.cuda.synchronize()
        ref_sol, ref_hist, ref_cky = R.tv_forward_history(I["wx"], I["wy"], I["c"], I["b"], I["init"], its)
        assert_close(sol, ref_sol, "solution")
        # the reverse sweep is compared on the iterates of a full-history run of the same forward pass (bit-identical)
        ext.set_option(pid, _lib.OPT_RECOMPUTE, 0)
        ext.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, pid)
        hist, cky = ext.read_history(pid, D["b"], its)
        ref = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, None, hist=hist.cpu(), ckpt_y=cky.cpu())
        for name, g, r in zip(GRAD_NAMES, grads, ref):
            assert_close(g, r, name)
    finally:
        ext.set_option(pid, _lib.OPT_RECOMPUTE, 0)
        ext.set_option(pid, _lib.OPT_CONDITIONER, 1)
        ext.release(pid)
