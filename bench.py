#!/usr/bin/env python
"""Benchmark of the TV-FISTA inpainting layer (forward + hand-derived backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling weak|strong]

One "step" = forward + backward of one batch of synthetic flow fields (2 x 384 x 1280, 100 iterations), plus the
lambda-gradient reduction and, on more than one GPU, its NCCL all-reduce.  The batch of 8 is sharded over the GPUs
(8/4/2/1 images per GPU at 1/2/4/8 GPUs: strong scaling, the default); `--scaling weak` keeps 8 images per GPU, and a
multi-GPU strong run carries that figure in `weak_scaling`.  Metric: Gpixel-iters/s = N*H*W*its_eff / t / 1e9.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "tv_fista_fwd_bwd_gpixel_iters_per_s"
UNIT = "Gpixel-iters/s"
WORKLOADS = {
    # name: (per-GPU batch, channels, height, width, iterations)
    "cfg1": (8, 2, 384, 1280, 100),
    "cfg0": (1, 2, 96, 320, 20),
    "small": (2, 2, 384, 1280, 20),      # profiling case: a few hundred MB on the device
    "odd": (8, 2, 375, 1242, 100),        # rows of 1242 floats: not a multiple of four, runs on zero-padded staging copies
    "prof": (8, 2, 384, 1280, 20),       # profiling case with the launch geometry of cfg1 and a fifth of its history
    "cfg2": (8, 2, 436, 1024, 100),      # TGV-FISTA (secondary workload, run with --workload cfg2)
    "cfg2small": (2, 2, 436, 1024, 10),  # TGV profiling case
    "cfg2prof": (8, 2, 436, 1024, 6),    # TGV profiling case with the launch geometry of cfg2 (persistent kernels)
    "cfg4": (32, 2, 384, 1280, 0),        # learnable 7x7 weighted-median filter (no iterations)
    "cfg4small": (2, 2, 384, 1280, 0),    # weighted-median profiling case
    "median": (4, 49, 384, 1280, 0),      # the reference's selection layer on a materialised [N,H,W,K] weight volume
    "quadfit": (4, 32, 384, 1280, 0),     # the reference's quadratic fit on two feature maps and a flow
    "cfg3": (16, 2, 512, 960, 50),       # coarse-to-fine stack of three TV layers (ids 0,1,2) with quadratic-fit refinement
}
CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def algorithmic_bytes_per_pixel_iter(ch: int):
    """Un-blocked schedule with the history stored once: forward (6C+3) floats, reverse (9C+9) floats."""
    return (6 * ch + 3) * 4, (9 * ch + 9) * 4


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = f"/tmp/cnl_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={CLOCK_QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle port (the reference is CUDA-only and cannot be built without ImageUtilities)
# ---------------------------------------------------------------------------------------------------------------
def cpu_fwd_bwd(I, its):
    import torch
    from oracle import tv_ref as R
    sol, ck = R.tv_forward_raw(I["wx"], I["wy"], I["c"], I["b"], I["init"], its, torch.float32)
    R.tv_backward_raw(I["wx"], I["wy"], I["c"], I["b"], I["grad"], its, ck, torch.float32)
    return sol


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per image and iteration of the single-launch sweeps at
# 2x384x1280, from an `ncu --set full` capture of one launch each on the `prof` workload (batch 8, 20 iterations:
# reverse 2654 MB for 19 iterations, forward 1693 MB for 20), NOT measured in this run
# (summary under profiles/).  Traffic grows in proportion to images and iterations of a launch, so
# other batch sizes and iteration counts of the same image scale it; other image sizes have no capture and report null.
NCU_TRAFFIC_PER_IMAGE_ITER = {(2, 384, 1280): {"reverse": 2653.8e6 / 19 / 8, "forward": 1693.2e6 / 20 / 8}}
TRAFFIC_SOURCE = ("ncu capture of one single-launch sweep on the prof workload (summary under profiles/), "
                  "scaled by images and iterations of the launch; not measured in this run")


def ncu_traffic_per_launch(nb, ch, h, w, rev_ipl, fwd_ipl):
    t = NCU_TRAFFIC_PER_IMAGE_ITER.get((ch, h, w))
    if not t:
        return None
    return {"reverse": t["reverse"] * nb * rev_ipl, "forward": t["forward"] * nb * fwd_ipl}


def cpu_baseline_sample(ch, h, w, its, budget_s=20.0):
    """Times the fp32 oracle on one image of the workload (cropped if a probe says it would exceed the budget)."""
    import torch
    from customnetworklayers_b200.synthetic import make_inputs
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ph, pw, pits = min(h, 96), min(w, 320), min(its, 20)
    I = make_inputs(1, ch, ph, pw, seed=1234)
    cpu_fwd_bwd(I, pits)
    t0 = time.perf_counter()
    cpu_fwd_bwd(I, pits)
    rate = ph * pw * 2 * (pits // 2) / (time.perf_counter() - t0)          # pixel-iters / s
    sh, sw = h, w
    while sh * sw * 2 * (its // 2) / rate > budget_s and sh > 32:
        sh //= 2
    I = make_inputs(1, ch, sh, sw, seed=1235)
    images, dt = 0, 0.0
    t0 = time.perf_counter()
    while dt < 12.0 and images < 64:             # one image at a time (the reference's calling pattern) for >= 12 s
        cpu_fwd_bwd(I, its)
        images += 1
        dt = time.perf_counter() - t0
    val = images * sh * sw * 2 * (its // 2) / dt / 1e9
    return {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"fp32 torch-CPU oracle, {images} x (1 image {ch}x{sh}x{sw}, {its} iterations, fwd+bwd) after a warm-up probe, {dt:.1f} s"}


def reference_cuda_sample(ch, h, w, its):
    """The reference's OWN cudaTV kernels (oracle/_ref/libtvref.so, built unmodified against a small ImageUtilities
    stand-in) timed on this GPU: one image per call is all the reference supports.  None if not built."""
    try:
        from oracle import ref_cuda
        if not ref_cuda.available() or h % 16 or w % 32:
            return None
        import torch
        from customnetworklayers_b200.synthetic import make_inputs
        I = make_inputs(1, ch, h, w, seed=1236)
        D = {k: v.cuda() for k, v in I.items()}

        def once():
            ref_cuda.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, 9)
            ref_cuda.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, 9)

        once()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        reps = 2
        for _ in range(reps):
            once()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / reps
        return {"value": h * w * 2 * (its // 2) / dt / 1e9, "unit": UNIT, "ms_per_image": dt * 1e3,
                "sample": f"reference cudaTV kernels (unmodified, sm_100a build), 1 image {ch}x{h}x{w}, {its} iterations, "
                          "fwd+bwd, host wall clock around its blocking calls (its checkpoints go through host memory)"}
    except Exception as e:          # the second checker is optional
        return {"unavailable": str(e)[:200]}


def workload_config(args, world):
    """The `config` block both arms print: names the workload, not the arm."""
    nb, ch, h, w, its = WORKLOADS[args.workload]
    scaling = resolve_scaling(args)
    gb = nb if scaling == "strong" else nb * world
    return {"workload": f"{args.workload}: TV-FISTA fwd+bwd, batch {gb}, flow {ch}x{h}x{w}, {its} iterations, "
                        f"sharded over {world} GPU(s), lambda gradient all-reduced",
            "global_batch": gb, "parallelism": f"dp{world}",
            "l2": "per-step working set (iterate history) is far larger than the 126 MB L2; no flush"}


def resolve_scaling(args):
    return args.scaling or "strong"


def run_reference_arm(args, rank, world):
    """--impl reference: the reference math on the host cores (oracle port, all threads), same metric and config.
    One step = forward + backward of ONE full image of the workload (the reference's own calling pattern is one image
    per call); the metric is per pixel-iteration, so the number compares directly."""
    if rank != 0:
        return
    import torch
    from customnetworklayers_b200.synthetic import make_inputs
    nb, ch, h, w, its = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    its_eff = 2 * (its // 2)
    I = make_inputs(1, ch, h, w, seed=1235)
    for _ in range(args.warmup):
        cpu_fwd_bwd(I, its)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_fwd_bwd(I, its)
    dt = time.perf_counter() - t0
    val = args.steps * h * w * its_eff / dt / 1e9
    sample = (f"fp32 torch-CPU oracle port on {cores} threads; per step 1 full image {ch}x{h}x{w}, {its} iterations, fwd+bwd "
              f"(1/{nb} of the batch: the reference solves one image per call)")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": resolve_scaling(args), "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(args, world),
            "arm": {"what": "the reference is CUDA-only and does not build without ImageUtilities; this arm times its CPU "
                            "restatement (oracle/tv_ref.py, float32)", "step": sample},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------
def measure_tv(args, dev, rank, local_rank, world, nb, ch, h, w, its, steps, warmup, sample_clocks, peer=None):
    """Times `steps` forward+backward steps of a per-GPU batch of nb images, inputs resident, then the same through the
    host-buffer API.  Returns a dict of raw figures (times are the maximum over ranks)."""
    import torch
    import torch.distributed as dist
    from customnetworklayers_b200 import _lib, tvInpaint_cuda_ext as ext
    from customnetworklayers_b200.dist import allreduce_scalar_grads
    from customnetworklayers_b200.host_pipeline import HostPipeline, tv_fwd_bwd_from_host
    from customnetworklayers_b200.synthetic import make_inputs

    pid = 0
    ext.release(pid)
    ext.set_option(pid, _lib.OPT_FUSE, args.fuse)
    ext.set_option(pid, _lib.OPT_RECOMPUTE, 1 if args.recompute else 0)
    ext.set_option(pid, _lib.OPT_CONDITIONER, 1)
    # seeded synthetic inputs; every rank draws its own shard
    I = make_inputs(nb, ch, h, w, seed=1234 + 1 + 1000 * rank)
    keys = ("wx", "wy", "c", "b", "init", "grad")
    host = {k: I[k].pin_memory() for k in keys}
    D = {k: host[k].to(dev, non_blocking=True) for k in keys}
    lam = torch.ones(1, device=dev)
    c_raw = D["c"]
    torch.cuda.synchronize()

    def step_resident():
        c = c_raw * lam                                   # c = lambda * c_raw, lambda is the learned scalar
        sol = ext.forward(D["wx"], D["wy"], c, D["b"], D["init"], its, pid)[0]
        grads = ext.backward(D["grad"], D["wx"], D["wy"], c, D["b"], its, pid)
        if peer is not None:                              # local reduction + exchange over peer memory, fused
            g_lam = peer.lambda_grad(grads[2], c_raw)
        else:
            g_lam = ext.lambda_grad(grads[2], c_raw)
            allreduce_scalar_grads(g_lam)
        return sol, grads, g_lam

    host_lam = torch.empty(1).pin_memory()
    pipe = HostPipeline(dev)
    out_keys = ("sol", "g_wx", "g_wy", "g_c", "g_b", "g_init")
    like = {"sol": "b", "g_wx": "wx", "g_wy": "wy", "g_c": "c", "g_b": "b", "g_init": "b"}
    host_res = {k: torch.empty_like(host[like[k]]).pin_memory() for k in out_keys}
    chunk = max(1, min(args.e2e_chunk, nb))

    def step_e2e():
        # the public host-buffer API: chunked H2D copy -> forward -> backward -> D2H copy, copies overlapped
        tv_fwd_bwd_from_host(pipe, host, host_res, its, pid, lam=lam, chunk=chunk, host_lam_grad=host_lam)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, nsteps, clocks=False, finish=None):
        barrier()
        sampler = ClockSampler(local_rank) if clocks else None
        if sampler:
            sampler.start()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        launches0 = _lib.load().cnl_launch_count()
        marks = []
        e0.record()
        for _ in range(nsteps):
            fn()
            m = torch.cuda.Event(enable_timing=True)
            m.record()
            marks.append(m)
        if finish:
            finish()                  # the timed stream waits for the last result copy before the closing event
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        launches = _lib.load().cnl_launch_count() - launches0
        per_step = [a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks)]      # compute-stream time between steps
        timed.last_per_step = per_step
        return float(ms.item()), launches, (sampler.stop() if sampler else None)

    for _ in range(warmup):
        step_resident()
    ext.set_option(pid, _lib.OPT_TIMING, 1)
    ms, launches, clocks = timed(step_resident, steps, clocks=sample_clocks)
    tm = ext.get_timing(pid)
    ext.set_option(pid, _lib.OPT_TIMING, 0)
    for _ in range(max(3, min(3, warmup))):
        step_e2e()
    ms_e2e, _, _ = timed(step_e2e, steps, finish=pipe.join)
    e2e_steps = sorted(timed.last_per_step)
    # where an end-to-end step spends its time: one call alone, CUDA events per chunk from the call's start
    # The same copies without any kernel: what the host memory / PCIe side of the box sustains when every rank streams
    # at once (the ceiling of the end-to-end figure on more than one GPU).
    copies_ms = None
    if world > 1:
        dbuf = {k: torch.empty_like(host[k], device=dev) for k in keys}
        obuf = {k: torch.empty_like(host_res[k], device=dev) for k in out_keys}

        def copies():
            with torch.cuda.stream(pipe.s_in):
                for k in keys:
                    dbuf[k].copy_(host[k], non_blocking=True)
            with torch.cuda.stream(pipe.s_out):
                for k in out_keys:
                    host_res[k].copy_(obuf[k], non_blocking=True)

        for _ in range(3):
            copies()
        barrier()
        c0, c1, c2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        c0.record()
        pipe.s_in.wait_event(c0)
        pipe.s_out.wait_event(c0)
        for _ in range(steps):
            copies()
        c1.record(pipe.s_in)
        c2.record(pipe.s_out)
        barrier()
        t = torch.tensor([max(c0.elapsed_time(c1), c0.elapsed_time(c2))], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        copies_ms = float(t.item()) / steps
        del dbuf, obuf
    barrier()
    pipe.timeline = []
    step_e2e()                        # on every rank: the call contains the all-reduce
    torch.cuda.synchronize()
    breakdown = [{k: round(v, 3) for k, v in row.items()} for row in pipe.chunk_breakdown()]
    pipe.timeline = None
    barrier()
    res = {"nb": nb, "ms": ms, "launches": launches, "clocks": clocks, "tm": tm, "ms_e2e": ms_e2e, "chunk": chunk,
           "h2d": sum(host[k].numel() * 4 for k in keys), "d2h": sum(t.numel() * 4 for t in host_res.values()) + 4,
           "breakdown": breakdown, "copies_ms": copies_ms,
           "e2e_step_ms": {"min": e2e_steps[0], "median": e2e_steps[len(e2e_steps) // 2], "max": e2e_steps[-1]}}
    del D, host, host_res, pipe
    ext.release(pid)
    torch.cuda.empty_cache()
    return res


def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    from customnetworklayers_b200 import _lib

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    _lib.load()

    nb_full, ch, h, w, its = WORKLOADS[args.workload]
    scaling = resolve_scaling(args)
    nb = nb_full
    if scaling == "strong":
        if nb_full % world:
            raise RuntimeError("strong scaling needs the batch to divide by the number of GPUs")
        nb = nb_full // world
    if args.per_gpu_batch:
        nb = args.per_gpu_batch          # one GPU standing in for one rank of a larger job (development aid)
    its_eff = 2 * (its // 2)
    peer, collective = None, "none (one GPU)"
    if world > 1:
        collective = "NCCL all-reduce of the lambda gradient (1 float)"
        if args.collective == "peer":
            try:
                from customnetworklayers_b200.dist import PeerAllReduce
                peer = PeerAllReduce()
                collective = "lambda-gradient reduction fused with a one-shot exchange over NVLink peer memory (cnl_tv_lambda_grad_allreduce)"
            except Exception as e:          # e.g. no symmetric-memory support: NCCL does the same job
                peer = None
                if rank == 0:
                    print(f"peer all-reduce unavailable ({str(e)[:160]}); using NCCL", file=sys.stderr, flush=True)
        # every rank must take the same path
        flag = torch.tensor([1 if peer is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            peer, collective = None, "NCCL all-reduce of the lambda gradient (1 float)"
    M = measure_tv(args, dev, rank, local_rank, world, nb, ch, h, w, its, args.steps, args.warmup, True, peer=peer)
    weak = None
    if world > 1 and scaling == "strong" and not args.per_gpu_batch:
        weak = measure_tv(args, dev, rank, local_rank, world, nb_full, ch, h, w, its, args.steps, args.warmup, False, peer=peer)

    ms, ms_e2e, tm = M["ms"], M["ms_e2e"], M["tm"]
    pixel_iters = world * nb * h * w * its_eff
    value = pixel_iters * args.steps / (ms * 1e-3) / 1e9
    e2e_value = pixel_iters * args.steps / (ms_e2e * 1e-3) / 1e9

    if rank == 0:
        fwd_b, rev_b = algorithmic_bytes_per_pixel_iter(ch)
        peak, peak_kind = measured_peak_gbs()
        # dominant kernel: the reverse iteration.  Average launch duration from CUDA events bracketing the reverse
        # loop of every timed step, on the stream the kernels run on.
        rev_launch_ms = tm["rev_ms"] / max(1, tm["rev_launches"])
        iters_per_launch = tm["rev_iters"] / max(1, tm["rev_launches"])
        bytes_per_launch = rev_b * nb * h * w * iters_per_launch
        achieved = bytes_per_launch / (rev_launch_ms * 1e-3) / 1e9 if rev_launch_ms > 0 else 0.0
        fwd_launch_ms = tm["fwd_ms"] / max(1, tm["fwd_launches"])
        fwd_ipl = tm["fwd_iters"] / max(1, tm["fwd_launches"])
        fwd_achieved = fwd_b * nb * h * w * fwd_ipl / (fwd_launch_ms * 1e-3) / 1e9 if fwd_launch_ms > 0 else 0.0
        whole = (fwd_b + rev_b) * pixel_iters / world * args.steps / (ms * 1e-3) / 1e9
        traffic = ncu_traffic_per_launch(nb, ch, h, w, iters_per_launch, fwd_ipl) if args.fuse in (0, 4) else None
        cfg = workload_config(args, world)
        if args.per_gpu_batch:
            cfg["workload"] += f" [one GPU timing a shard of {nb} image(s)]"
            cfg["global_batch"] = nb
        arm = {"what": "this library on the GPU(s)", "per_gpu_batch": nb, "fuse": args.fuse, "collective": collective,
               "history": "checkpoints only, segments recomputed in the backward pass" if args.recompute else "every iterate resident"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg, "arm": arm,
            "roofline": {"bound": "hbm", "kernel": "reverse sweep (tv_rev_flow_kernel: every full 4-iteration time block in one launch)" if iters_per_launch > 4 else "reverse iteration kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic["reverse"] if traffic else None,
                         "frac_traffic": (traffic["reverse"] / (rev_launch_ms * 1e-3) / 1e9 / peak) if traffic and rev_launch_ms > 0 else None,
                         "traffic_source": TRAFFIC_SOURCE if traffic else None,
                         "peak_kind": peak_kind, "limiter": "instruction issue, not DRAM: see frac_traffic",
                         "launch_ms": rev_launch_ms, "iterations_per_launch": iters_per_launch,
                         "algorithmic_bytes_per_launch": bytes_per_launch,
                         "note": "achieved counts the bytes a one-iteration-per-launch schedule streams; fused iterations "
                                 "move about a third of that through DRAM (traffic), hence frac > 1 while frac_traffic, "
                                 "the share of the copy peak the launch really draws, is well below 1",
                         "forward_kernel": {"achieved": fwd_achieved, "frac": fwd_achieved / peak, "launch_ms": fwd_launch_ms,
                                            "iterations_per_launch": fwd_ipl,
                                            "traffic": traffic["forward"] if traffic else None,
                                            "frac_traffic": (traffic["forward"] / (fwd_launch_ms * 1e-3) / 1e9 / peak) if traffic and fwd_launch_ms > 0 else None},
                         "whole_step": {"achieved": whole, "frac": whole / peak}},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": M["h2d"], "d2h_bytes_per_step": M["d2h"],
                    "ms_per_step": ms_e2e / args.steps, "api": "host_pipeline.tv_fwd_bwd_from_host",
                    "chunk_images": M["chunk"],
                    "step_ms_on_compute_stream": M["e2e_step_ms"],
                    "copies_only_ms_per_step": M["copies_ms"],
                    "copies_only_aggregate_gbs": ((M["h2d"] + M["d2h"]) * world / (M["copies_ms"] * 1e-3) / 1e9) if M["copies_ms"] else None,
                    "single_call_ms_since_start": M["breakdown"]},
            "gpu_launches": int(M["launches"]),
            "clocks": M["clocks"],
        }
        if weak is not None:
            wpi = world * nb_full * h * w * its_eff
            line["weak_scaling"] = {"per_gpu_batch": nb_full, "global_batch": nb_full * world,
                                    "value": wpi * args.steps / (weak["ms"] * 1e-3) / 1e9, "ms_per_step": weak["ms"] / args.steps,
                                    "e2e_value": wpi * args.steps / (weak["ms_e2e"] * 1e-3) / 1e9,
                                    "e2e_ms_per_step": weak["ms_e2e"] / args.steps, "unit": UNIT}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample(ch, h, w, its)
            rc = reference_cuda_sample(ch, h, w, its)
            if rc is not None:
                line["reference_cuda"] = rc
        if world == 1 and not args.no_secondary and args.workload == "cfg1" and not args.per_gpu_batch:
            line["secondary"] = secondary_workloads(args, local_rank)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def secondary_workloads(args, local_rank):
    """Compact records of the other configurations (TGV, the coarse-to-fine stack, the weighted-median filter and the two
    small layers), three steps each after three warm-up steps, measured after and outside the timed region above."""
    import copy
    out = {}
    for name, fn in (("cfg2", run_tgv), ("cfg3", run_hierarchy), ("cfg4", run_wmedian), ("median", run_layer_micro),
                     ("quadfit", run_layer_micro)):
        a = copy.copy(args)
        a.workload, a.steps, a.warmup = name, 3, 3
        try:
            r = fn(a, 0, local_rank, 1)
            out[name] = {"metric": r["metric"], "value": r["value"], "unit": r["unit"], "ms_per_step": r["ms_per_step"],
                         "frac": r["roofline"]["frac"], "roofline_kernel": r["roofline"]["kernel"],
                         "workload": r["config"]["workload"], "gpu_launches": r["gpu_launches"]}
        except Exception as e:          # a secondary record must not take the headline down with it
            out[name] = {"error": str(e)[:200]}
    return out


def run_tgv(args, rank, local_rank, world):
    """Secondary workload: TGV-FISTA fwd+bwd (batch 8 per GPU, 2x436x1024, 100 iterations); same JSON contract, the
    roofline entry is the whole step against 376 B per pixel-iteration ((16C+5)*4 forward + (21C+15)*4 reverse)."""
    import torch
    import torch.distributed as dist
    from customnetworklayers_b200 import _lib, tgvInpaint_cuda_ext as ext
    from customnetworklayers_b200.dist import allreduce_scalar_grads
    from customnetworklayers_b200.synthetic import make_tgv_inputs
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    nb, ch, h, w, its = WORKLOADS[args.workload]
    its_eff = 2 * (its // 2)
    I = make_tgv_inputs(nb, ch, h, w, seed=1236 + 1000 * rank)
    D = {k: v.to(dev) for k, v in I.items()}
    flat = lambda t: t.reshape(nb, 3 * ch, h, w)
    alpha = torch.tensor([1.0, 2.0], device=dev)          # learned scalars alpha0 (edge weights), alpha1 (beta)
    pid = 1

    def step():
        sol = ext.forward(D["dx"], D["dy"], D["c"], D["b"], flat(D["init"]), its, pid)[0]
        g = ext.backward(flat(D["grad"]), D["dx"], D["dy"], D["c"], D["b"], its, pid)
        # d/d alpha_k = sum over pixels of grad * raw map; dx = [alpha0*wx, alpha1*1]
        g_alpha = torch.stack([(g[0][:, 0] * D["dx"][:, 0]).sum() + (g[1][:, 0] * D["dy"][:, 0]).sum(),
                               (g[0][:, 1] * D["dx"][:, 1]).sum() + (g[1][:, 1] * D["dy"][:, 1]).sum()]) / alpha
        allreduce_scalar_grads(g_alpha)
        return sol, g_alpha

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = _lib.load().cnl_launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    launches = _lib.load().cnl_launch_count() - l0
    clocks = sampler.stop()
    result = None
    if rank == 0:
        pixel_iters = world * nb * h * w * its_eff
        value = pixel_iters * args.steps / (ms * 1e-3) / 1e9
        bytes_pi = (16 * ch + 5) * 4 + (21 * ch + 15) * 4
        peak, kind = measured_peak_gbs()
        ach = bytes_pi * pixel_iters / world * args.steps / (ms * 1e-3) / 1e9
        result = ({
            "metric": "tgv_fista_fwd_bwd_gpixel_iters_per_s", "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cfg2: TGV-FISTA fwd+bwd, per-GPU batch {nb}, flow {ch}x{h}x{w} + 2 auxiliary planes per channel, {its} iterations, alpha gradients all-reduced",
                       "global_batch": nb * world, "parallelism": f"dp{world}"},
            "roofline": {"bound": "hbm", "kernel": "whole step (one launch per iteration)", "achieved": ach, "peak": peak,
                         "unit": "GB/s", "frac": ach / peak, "traffic": None, "peak_kind": kind},
            "gpu_launches": int(launches), "clocks": clocks})
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def run_hierarchy(args, rank, local_rank, world):
    """Secondary workload: three TV layers at 1/4, 1/2 and full resolution (ids 0, 1, 2; 50 iterations each), a
    quadratic-fit refinement before each level, bilinear x2 upsampling between levels, full fwd+bwd; the three lambda
    gradients are all-reduced.  Metric counts the TV pixel-iterations of all levels."""
    import torch
    import torch.distributed as dist
    from customnetworklayers_b200 import _lib
    from customnetworklayers_b200.hierarchical import HierarchicalTV
    from customnetworklayers_b200.synthetic import make_hierarchy_inputs
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    nb, ch, h, w, its = WORKLOADS[args.workload]
    its_eff = 2 * (its // 2)
    levels, grad = make_hierarchy_inputs(nb, h, w, seed=1237 + 1000 * rank)
    D = [{k: v.to(dev).requires_grad_(k == "cost5") for k, v in I.items()} for I in levels]
    grad = grad.to(dev)
    model = HierarchicalTV(levels=3, its=its).to(dev)

    def step():
        model.zero_grad(set_to_none=True)
        for d in D:
            d["cost5"].grad = None
        sols = model(D)
        sols[-1].backward(grad)
        model.allreduce_parameter_grads()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = _lib.load().cnl_launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    launches = _lib.load().cnl_launch_count() - l0
    clocks = sampler.stop()
    result = None
    if rank == 0:
        pixel_iters = world * nb * sum((h >> s) * (w >> s) for s in (2, 1, 0)) * its_eff
        value = pixel_iters * args.steps / (ms * 1e-3) / 1e9
        peak, kind = measured_peak_gbs()
        fwd_b, rev_b = algorithmic_bytes_per_pixel_iter(ch)
        ach = (fwd_b + rev_b) * pixel_iters / world * args.steps / (ms * 1e-3) / 1e9
        result = ({
            "metric": "hierarchical_tv_fwd_bwd_gpixel_iters_per_s", "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cfg3: 3-level TV stack (ids 0,1,2), per-GPU batch {nb}, flow {ch}x{h}x{w}, {its} iterations per level, quadratic-fit refinement and bilinear upsampling between levels",
                       "global_batch": nb * world, "parallelism": f"dp{world}"},
            "roofline": {"bound": "hbm", "kernel": "whole step (TV pixel-iterations only)", "achieved": ach, "peak": peak,
                         "unit": "GB/s", "frac": ach / peak, "traffic": None, "peak_kind": kind},
            "gpu_launches": int(launches), "clocks": clocks})
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def run_wmedian(args, rank, local_rank, world):
    """Secondary workload: learnable 7x7 weighted-median filter fwd+bwd, batch 32 per GPU, flow 2x384x1280 with 5 %
    outliers; the 49 weight gradients are all-reduced.  Metric: median problems (pixel-channels) per second."""
    import torch
    import torch.distributed as dist
    from customnetworklayers_b200 import _lib
    from customnetworklayers_b200.synthetic import make_median_filter_inputs
    from customnetworklayers_b200.wmedian import WeightedMedianFilter
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    nb, ch, h, w, _ = WORKLOADS[args.workload]
    flow, wts, grad = make_median_filter_inputs(nb, ch, h, w, seed=1238 + 1000 * rank)
    flow, grad = flow.to(dev), grad.to(dev)
    model = WeightedMedianFilter(7).to(dev)
    with torch.no_grad():
        model.weight.copy_(wts)

    def step():
        model.zero_grad(set_to_none=True)
        x = flow.detach().requires_grad_(True)
        model(x).backward(grad)
        model.allreduce_parameter_grads()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = _lib.load().cnl_launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    launches = _lib.load().cnl_launch_count() - l0
    clocks = sampler.stop()
    result = None
    if rank == 0:
        problems = world * nb * ch * h * w
        value = problems * args.steps / (ms * 1e-3) / 1e9
        peak, kind = measured_peak_gbs()
        # fused layout: read flow + grad, write out + tap + g_flow, re-read tap + grad: 7 words per problem; the
        # reference's materialised layout would move (3*49+4)*4 = 604 B per problem
        ach = 28.0 * problems / world * args.steps / (ms * 1e-3) / 1e9
        result = ({
            "metric": "weighted_median_fwd_bwd_gproblems_per_s", "value": value, "unit": "Gproblems/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cfg4: learnable 7x7 weighted-median filter fwd+bwd, per-GPU batch {nb}, flow {ch}x{h}x{w}, 5% outliers, 49 weight gradients all-reduced",
                       "global_batch": nb * world, "parallelism": f"dp{world}"},
            "roofline": {"bound": "hbm", "kernel": "whole step; the kernels are bound by instruction issue in the rank updates of the sliding window (k*(K-k) compares and twice as many adds per problem), not by HBM",
                         "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None, "peak_kind": kind,
                         "materialised_layout_equivalent_gbs": 604.0 * problems / world * args.steps / (ms * 1e-3) / 1e9},
            "gpu_launches": int(launches), "clocks": clocks})
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def run_layer_micro(args, rank, local_rank, world):
    """Micro workloads for the two remaining reference layers, through their extension modules: `median` (selection on
    a materialised [N,H,W,K] volume, (3K+4)*4 B per problem fwd+bwd) and `quadfit` (features + flow API,
    (7C+10)*4 B per pixel fwd+bwd: forward reads both feature maps once and the flow, writes 3 planes; backward
    reads them again with the upstream gradient, zero-fills and writes both feature gradients).  One GPU each."""
    import torch
    from customnetworklayers_b200 import _lib
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    nb, k, h, w, _ = WORKLOADS[args.workload]
    if args.workload == "median":
        from customnetworklayers_b200 import median_cuda_ext as ext
        from customnetworklayers_b200.synthetic import make_median_volume
        vol, grad = make_median_volume(nb, h, w, k, seed=1238 + rank)
        vol, grad = vol.to(dev), grad.to(dev)
        step = lambda: (ext.forward(vol), ext.backward(grad, vol))
        units, bytes_per_unit = nb * h * w, (3 * k + 4) * 4
        metric, unit, what = "median_fwd_bwd_gproblems_per_s", "Gproblems/s", f"selection on a [N,H,W,{k}] weight volume"
    else:
        from customnetworklayers_b200 import QuadFit_cuda_ext as ext
        from customnetworklayers_b200.synthetic import make_quadfit_inputs
        f0, f1, flow, grad = (t.to(dev) for t in make_quadfit_inputs(nb, k, h, w, seed=1237 + rank))
        step = lambda: (ext.forward(f0, f1, flow), ext.backward(grad, f0, f1, flow))
        units, bytes_per_unit = nb * h * w, (7 * k + 10) * 4
        metric, unit, what = "quadfit_fwd_bwd_gpixels_per_s", "Gpixels/s", f"quadratic fit on {k}-channel feature maps"
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = _lib.load().cnl_launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = _lib.load().cnl_launch_count() - l0
    clocks = sampler.stop()
    result = None
    if rank == 0:
        peak, kind = measured_peak_gbs()
        ach = bytes_per_unit * units * args.steps / (ms * 1e-3) / 1e9
        result = ({
            "metric": metric, "value": units * args.steps / (ms * 1e-3) / 1e9, "unit": unit, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {what}, batch {nb}, {h}x{w}, fwd+bwd",
                       "l2": "inputs of several hundred MB per call, larger than the 126 MB L2; no flush"},
            "roofline": {"bound": "hbm", "kernel": "whole step", "achieved": ach, "peak": peak, "unit": "GB/s",
                         "frac": ach / peak, "traffic": None, "peak_kind": kind, "algorithmic_bytes_per_unit": bytes_per_unit},
            "gpu_launches": int(launches), "clocks": clocks})
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="strong (default): the batch of the workload is sharded over the GPUs; weak: that batch per GPU")
    ap.add_argument("--per-gpu-batch", type=int, default=0,
                    help="development aid: time this many images on the GPU(s) given, as one rank of a larger job would")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="how the lambda gradient is summed over GPUs: fused reduction + exchange over peer memory, or NCCL")
    ap.add_argument("--no-secondary", action="store_true", help="skip the compact records of the other configurations")
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--fuse", type=int, default=0)
    ap.add_argument("--recompute", action="store_true",
                    help="keep only checkpoints on the device and rebuild the iterate history segment by segment in the backward pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunk", type=int, default=4, help="images per chunk of the host-buffer pipeline")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # launched without torchrun: re-launch as one process per GPU
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29513"),
                   os.path.abspath(__file__)] + sys.argv[1:]
            sys.exit(subprocess.call(cmd))
        raise RuntimeError(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    result = None
    if args.workload in ("median", "quadfit"):
        if rank == 0:
            result = run_layer_micro(args, rank, local_rank, world)
    elif args.workload.startswith("cfg4"):
        result = run_wmedian(args, rank, local_rank, world)
    elif args.workload == "cfg3":
        result = run_hierarchy(args, rank, local_rank, world)
    elif args.workload.startswith("cfg2"):
        result = run_tgv(args, rank, local_rank, world)
    else:
        run_ours(args, rank, local_rank, world)
    if result is not None:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
