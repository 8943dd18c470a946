"""Data-parallel plumbing of the layer: the batch is sharded over ranks (one process per GPU) and the only
collective is a sum all-reduce of the learned-scalar gradients.  Uses torch.distributed (NCCL on GPUs, gloo in
CPU tests); images never cross ranks."""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch


def shard_range(n_items: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous shard [lo, hi) of `n_items` images for `rank` of `world`; sizes differ by at most one."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} / world {world}")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def allreduce_scalar_grads(g: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum of a small gradient vector (lambda for TV) over all ranks; no-op without a process group."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
    return g


def bind_to_gpu_numa_node(device_index: int) -> Optional[List[int]]:
    """Restricts the calling process to the CPUs NVML reports as closest to CUDA device `device_index`, so that pinned
    staging buffers allocated afterwards land (by first touch) in the host memory next to that GPU.  Matters when
    several ranks of one host stream to their GPUs at the same time.  Returns the CPU list, or None when nothing was
    changed (NVML unavailable, no overlap with the CPUs this process may use).  Reads NVML only; changes no GPU setting."""
    try:
        import pynvml
        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(device_index)
        bus_id = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (max(ncpu, 64) + 63) // 64 * 2)
        near = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus = sorted(near & allowed)
        if not cpus or len(cpus) == len(allowed):
            return None
        os.sched_setaffinity(0, cpus)
        return cpus
    except Exception:
        return None


class RankLeft(RuntimeError):
    """Raised by StepGuard.check() when another rank has announced that it stopped taking part."""


class StepGuard:
    """Host-side failure detection between steps for the batch-sharded layer.

    The only collective of the path is a tiny all-reduce per step, so a rank that stops (an exception in its data
    loader, a scale-down) would leave the others blocked in that all-reduce until the process-group timeout.  A rank
    that leaves cleanly calls leave() between steps, with none of its kernels or collectives in flight; every rank
    calls check() before it launches a step and gets RankLeft instead of a hang.  A rank that dies without saying so is
    caught by the process-group timeout of the next all-reduce (pass a short `timeout` to init_process_group).
    Uses a key-value store (torch.distributed.TCPStore or the like); no GPU is involved."""

    def __init__(self, store, rank: int, world: int):
        self.store, self.rank, self.world = store, rank, world

    def leave(self) -> None:
        self.store.set(f"cnl/left/{self.rank}", "1")

    def check(self) -> None:
        for r in range(self.world):
            if r != self.rank and self.store.check([f"cnl/left/{r}"]):
                raise RankLeft(f"rank {r} has left: stop before the next all-reduce")
