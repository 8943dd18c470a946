"""world_size-2 gloo test of the data-parallel plumbing: batch shards + the lambda-gradient all-reduce.
The per-shard layer math runs on the CPU oracle here (no GPU in this test); what is checked is the sharding and
the collective the GPU path uses unchanged."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from customnetworklayers_b200.dist import allreduce_scalar_grads, shard_range
    from oracle import tv_ref as R
    n, ch, h, w, its = 5, 2, 12, 16, 6
    I = R.make_inputs(n, ch, h, w, seed=3)
    lo, hi = shard_range(n, rank, world)
    S = {k: v[lo:hi] for k, v in I.items()}
    sol, ck = R.tv_forward_raw(S["wx"], S["wy"], S["c"], S["b"], S["init"], its)
    g = R.tv_backward_raw(S["wx"], S["wy"], S["c"], S["b"], S["grad"], its, ck)
    g_lam = (g[2] * S["c"].double()).sum().reshape(1)
    allreduce_scalar_grads(g_lam)
    q.put((rank, lo, hi, float(g_lam), sol.double().sum().item()))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_range_partitions_the_batch():
    from customnetworklayers_b200.dist import shard_range
    for n in (1, 5, 8, 16):
        for world in (1, 2, 3, 4, 8):
            parts = [shard_range(n, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            sizes = [hi - lo for lo, hi in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_two_ranks_allreduce_lambda_gradient():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    res.sort()
    assert (res[0][1], res[0][2], res[1][1], res[1][2]) == (0, 3, 3, 5)
    # every rank holds the same all-reduced value, equal to the single-process full-batch value
    assert abs(res[0][3] - res[1][3]) == 0.0
    sys.path.insert(0, ROOT)
    from oracle import tv_ref as R
    I = R.make_inputs(5, 2, 12, 16, seed=3)
    sol, ck = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], 6)
    g = R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], 6, ck)
    full = float((g[2] * I["c"].double()).sum())
    assert abs(res[0][3] - full) <= 1e-12 * max(1.0, abs(full))
    assert abs(res[0][4] + res[1][4] - sol.double().sum().item()) < 1e-9


def _guard_worker(rank, world, port, q):
    import datetime
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from customnetworklayers_b200.dist import RankLeft, StepGuard, allreduce_scalar_grads
    store = dist.TCPStore("127.0.0.1", port + 1, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    guard = StepGuard(store, rank, world)
    steps_done = 0
    try:
        for step in range(5):
            guard.check()
            g = torch.ones(1)
            allreduce_scalar_grads(g)
            assert float(g) == world
            steps_done += 1
            if rank == 1 and step == 1:          # this rank stops between steps, nothing in flight
                guard.leave()
                q.put((rank, "left", steps_done))
                return
            if rank == 0 and step == 1:          # give the announcement time to land before the next check
                import time
                for _ in range(200):
                    if store.check(["cnl/left/1"]):
                        break
                    time.sleep(0.05)
    except RankLeft as e:
        q.put((rank, "stopped: " + str(e), steps_done))
        return
    q.put((rank, "finished", steps_done))


def test_a_rank_that_leaves_between_steps_stops_the_others_without_a_hang():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_guard_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[1] == (1, "left", 2)
    assert res[0][0] == 0 and res[0][1].startswith("stopped: rank 1 has left") and res[0][2] == 2


def _silent_worker(rank, world, port, q):
    import datetime
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from customnetworklayers_b200.dist import allreduce_scalar_grads
    g = torch.ones(1)
    allreduce_scalar_grads(g)
    if rank == 1:
        q.put((rank, "gone"))
        q.close()
        q.join_thread()                           # the test wants to hear that this point was reached
        os._exit(0)                               # dies without a word to the other rank
    try:
        allreduce_scalar_grads(torch.ones(1))
        q.put((rank, "no error"))
    except Exception as e:                        # the short process-group timeout / the closed connection ends the wait
        q.put((rank, "error: " + type(e).__name__))


def test_a_rank_that_dies_silently_ends_the_next_all_reduce_with_an_error():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_silent_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert res[1] == "gone"
    assert res[0].startswith("error: ")
