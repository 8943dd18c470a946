"""The one-shot all-reduce over peer memory (cnl_peer_allreduce_sum, cnl_tv_lambda_grad_allreduce) on ONE GPU.

A second rank is stood in for by writing what it would have stored (value and call number in one 8-byte word) into this
rank's exchange buffer before the kernel starts, so nothing ever waits for another launch; the rank's own stores to its
"peer" go to a scratch buffer that is checked afterwards.  The real multi-GPU exchange is what `bench.py --gpus N` runs."""
import ctypes
import struct

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_WORLD, MAX_COUNT = 16, 64


def _slot(seq, from_rank, i):
    return ((seq & 1) * MAX_WORLD + from_rank) * MAX_COUNT + i


def _packed(seq, value):
    bits = struct.unpack("<I", struct.pack("<f", float(value)))[0]
    v = (seq << 32) | bits
    return v - (1 << 64) if v >= (1 << 63) else v          # as a signed int64 for torch


def _bufs(lib, n):
    words = lib.cnl_peer_allreduce_bytes() // 8
    assert words == 2 * MAX_WORLD * MAX_COUNT
    return [torch.zeros(words, dtype=torch.int64, device="cuda") for _ in range(n)]


def test_two_ranks_with_a_prefilled_peer_and_alternating_sets():
    from customnetworklayers_b200 import _lib
    lib = _lib.load()
    mine, theirs = _bufs(lib, 2)
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator().manual_seed(3)
    for seq in (1, 2, 3):                      # both sets, and a set reused with a newer call number
        count = (5, 64, 1)[seq - 1]
        a = torch.randn(count, generator=gen)
        b = torch.randn(count, generator=gen)
        for i in range(count):                 # what rank 1 would have stored into rank 0's buffer
            mine[_slot(seq, 1, i)] = _packed(seq, b[i])
        vals = a.cuda()
        _lib.check(lib.cnl_peer_allreduce_sum(vals.data_ptr(), count, ptrs, 0, 2, seq, st), "peer all-reduce")
        torch.cuda.synchronize()
        assert torch.equal(vals.cpu(), a + b), seq          # rank order: own value first, one rounding, exact match
        for i in range(count):                 # and rank 0's values arrived in the peer's buffer, tagged with the call
            assert int(theirs[_slot(seq, 0, i)]) == _packed(seq, a[i])
    assert lib.cnl_peer_allreduce_status() == 0


def test_fused_lambda_gradient_with_world_one_equals_the_plain_reduction():
    from customnetworklayers_b200 import _lib, tvInpaint_cuda_ext as ext
    lib = _lib.load()
    (mine,) = _bufs(lib, 1)
    ptrs = (ctypes.c_void_p * 1)(mine.data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    g = torch.randn(3 * 384 * 1280, device="cuda")
    c = torch.rand_like(g)
    ref = ext.lambda_grad(g, c)
    for seq in (1, 2):
        out = torch.full((1,), float("nan"), device="cuda")
        scratch = torch.empty(lib.cnl_dot_scratch_floats(), device="cuda")
        _lib.check(lib.cnl_tv_lambda_grad_allreduce(g.data_ptr(), c.data_ptr(), g.numel(), out.data_ptr(), scratch.data_ptr(),
                                                    ptrs, 0, 1, seq, st), "fused lambda gradient")
        torch.cuda.synchronize()
        assert torch.equal(out, ref)


def test_a_peer_that_never_answers_ends_in_nan_and_a_status_not_in_a_hang():
    from customnetworklayers_b200 import _lib
    lib = _lib.load()
    mine, theirs = _bufs(lib, 2)
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
    vals = torch.ones(2, device="cuda")
    _lib.check(lib.cnl_peer_allreduce_sum(vals.data_ptr(), 2, ptrs, 0, 2, 7, torch.cuda.current_stream().cuda_stream), "peer all-reduce")
    torch.cuda.synchronize()                    # returns: the wait is bounded
    assert bool(torch.isnan(vals).all())
    assert lib.cnl_peer_allreduce_status() == 7


def test_argument_checks():
    from customnetworklayers_b200 import _lib
    lib = _lib.load()
    (mine,) = _bufs(lib, 1)
    ptrs = (ctypes.c_void_p * 1)(mine.data_ptr())
    v = torch.ones(1, device="cuda")
    assert lib.cnl_peer_allreduce_sum(v.data_ptr(), 65, ptrs, 0, 1, 1, None) == 2
    assert lib.cnl_peer_allreduce_sum(v.data_ptr(), 1, ptrs, 1, 1, 1, None) == 2      # rank outside the world
    assert lib.cnl_peer_allreduce_sum(v.data_ptr(), 1, ptrs, 0, 1, 0, None) == 2      # call numbers start at 1
    assert lib.cnl_peer_allreduce_sum(None, 1, ptrs, 0, 1, 1, None) == 7


def _two_rank_worker(rank, world, port, q):
    import os
    import sys
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    from customnetworklayers_b200 import tvInpaint_cuda_ext as ext
    from customnetworklayers_b200.dist import PeerAllReduce
    peer = PeerAllReduce()
    gen = torch.Generator().manual_seed(100 + rank)
    ok = True
    for it in range(5):
        v = torch.randn(49, generator=gen).cuda()
        ref = v.clone()
        dist.all_reduce(ref)                                  # NCCL as the reference sum
        peer.sum_(v)
        ok = ok and bool(torch.allclose(v, ref, rtol=1e-6, atol=1e-6))
        g = torch.randn(100000, generator=gen).cuda()
        c = torch.rand(100000, generator=gen).cuda()
        ref1 = ext.lambda_grad(g, c)
        dist.all_reduce(ref1)
        out = peer.lambda_grad(g, c)
        ok = ok and bool(torch.allclose(out, ref1, rtol=1e-6, atol=1e-5))
    torch.cuda.synchronize()
    q.put((rank, ok, peer.status()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_two_real_ranks_agree_with_nccl():
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res == [(0, True, 0), (1, True, 0)]
