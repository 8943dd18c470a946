"""The allocation-free lambda-gradient entry point (cnl_tv_lambda_grad_static) against the scratch-taking one.

Some users of this library cannot allocate device memory at call time: a real-time loop that must avoid the
allocator's implicit synchronisation, or a plugin inside an engine that owns the whole device.  For them the
reduction's block partials sit in a fixed array inside the library.  This file is named to be collected last."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, a, b):
    from customnetworklayers_b200 import _lib
    st = torch.cuda.current_stream().cuda_stream
    ref = torch.empty(1, device="cuda")
    scratch = torch.empty(lib.cnl_dot_scratch_floats(), device="cuda")
    _lib.check(lib.cnl_tv_lambda_grad(a.data_ptr(), b.data_ptr(), a.numel(), ref.data_ptr(), scratch.data_ptr(), st),
               "lambda_grad")
    out = torch.full((1,), float("nan"), device="cuda")
    _lib.check(lib.cnl_tv_lambda_grad_static(a.data_ptr(), b.data_ptr(), a.numel(), out.data_ptr(), st),
               "lambda_grad_static")
    torch.cuda.synchronize()
    return float(out), float(ref)


def test_static_scratch_variant_matches_on_two_calls_in_a_row():
    from customnetworklayers_b200 import _lib
    lib = _lib.load()
    gen = torch.Generator().manual_seed(21)
    # first call: a large input that fills many slots; second call: a smaller, different input, so stale slots
    # from the first call would show up if they were read
    sizes = [8 * 384 * 1280, 3 * 1000 + 17]
    for n in sizes:
        a = torch.randn(n, generator=gen).cuda()
        b = torch.rand(n, generator=gen).cuda()
        got, ref = _both(lib, a, b)
        exact = float((a.double() * b.double()).sum())
        assert abs(got - ref) <= 1e-4 * max(1.0, abs(ref)), (n, got, ref)
        assert abs(got - exact) <= 1e-4 * max(1.0, abs(exact)), (n, got, exact)
    # and once more with the first size: same answer as a fresh computation
    a = torch.randn(sizes[0], generator=gen).cuda()
    b = torch.rand(sizes[0], generator=gen).cuda()
    got, ref = _both(lib, a, b)
    assert abs(got - ref) <= 1e-4 * max(1.0, abs(ref))


def test_static_variant_handles_empty_and_rejects_oversize():
    from customnetworklayers_b200 import _lib
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    a = torch.ones(4, device="cuda")
    out = torch.full((1,), 5.0, device="cuda")
    assert lib.cnl_tv_lambda_grad_static(a.data_ptr(), a.data_ptr(), 0, out.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert float(out) == 0.0
    too_many = lib.cnl_tv_lambda_grad_static_max_count() + 1
    rc = lib.cnl_tv_lambda_grad_static(a.data_ptr(), a.data_ptr(), too_many, out.data_ptr(), st)
    assert rc == 2 and "at most" in _lib.last_error()


def test_static_variant_at_its_maximum_count():
    """count == cnl_tv_lambda_grad_static_max_count() uses every slot of the array and must still be accepted."""
    from customnetworklayers_b200 import _lib
    lib = _lib.load()
    n = lib.cnl_tv_lambda_grad_static_max_count()
    gen = torch.Generator().manual_seed(22)
    a = torch.randn(n, generator=gen).cuda()
    b = torch.rand(n, generator=gen).cuda()
    for _ in range(2):
        got, ref = _both(lib, a, b)
        assert abs(got - ref) <= 1e-4 * max(1.0, abs(ref)), (got, ref)
