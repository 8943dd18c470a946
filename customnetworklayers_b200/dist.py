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


class PeerAllReduce:
    """All-reduce (sum) of a few floats over the GPUs of one node through peer memory instead of NCCL.

    The data-parallel layers exchange one to a few dozen scalars per step, for which a collective is pure latency.
    Each rank owns a small exchange buffer in symmetric memory (torch.distributed._symmetric_memory: the same
    allocation mapped into every process of the group); cnl_peer_allreduce_sum / cnl_tv_lambda_grad_allreduce let every
    rank store its values straight into its peers' buffers and sum what arrived in its own.  Collective: construct it on
    every rank of the group, after torch.cuda.set_device, and make the same calls in the same order on all ranks."""

    def __init__(self, group=None):
        import ctypes
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        self.lib = _lib.load()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        words = self.lib.cnl_peer_allreduce_bytes() // 8
        self.buf = symm_mem.empty(words, dtype=torch.int64, device=self.device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world:
            raise RuntimeError("symmetric memory rendezvous returned %d buffers for %d ranks" % (len(ptrs), self.world))
        self.peer_bufs = (ctypes.c_void_p * self.world)(*ptrs)
        self.seq = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)            # every buffer is zeroed before anyone stores into it

    def _next(self) -> int:
        self.seq += 1
        return self.seq

    def sum_(self, values: torch.Tensor) -> torch.Tensor:
        """In-place sum over all ranks of a contiguous float32 CUDA tensor of at most 64 elements."""
        from . import _lib
        if not (values.is_cuda and values.dtype == torch.float32 and values.is_contiguous()):
            raise RuntimeError("PeerAllReduce.sum_ needs a contiguous float32 CUDA tensor")
        rc = self.lib.cnl_peer_allreduce_sum(values.data_ptr(), values.numel(), self.peer_bufs, self.rank, self.world,
                                             self._next(), torch.cuda.current_stream(values.device).cuda_stream)
        _lib.check(rc, "peer all-reduce")
        return values

    def lambda_grad(self, g_c: torch.Tensor, c_raw: torch.Tensor, out=None, scratch=None) -> torch.Tensor:
        """sum over all ranks of sum(g_c * c_raw): the local reduction and the exchange in one kernel."""
        from . import _lib
        if out is None:
            out = torch.empty(1, dtype=torch.float32, device=g_c.device)
        if scratch is None:
            scratch = torch.empty(self.lib.cnl_dot_scratch_floats(), dtype=torch.float32, device=g_c.device)
        if not (g_c.is_cuda and c_raw.is_cuda and g_c.is_contiguous() and c_raw.is_contiguous()
                and g_c.dtype == torch.float32 and c_raw.dtype == torch.float32 and g_c.numel() == c_raw.numel()):
            raise RuntimeError("lambda_grad needs two contiguous float32 CUDA tensors of the same size")
        rc = self.lib.cnl_tv_lambda_grad_allreduce(g_c.data_ptr(), c_raw.data_ptr(), g_c.numel(), out.data_ptr(),
                                                   scratch.data_ptr(), self.peer_bufs, self.rank, self.world, self._next(),
                                                   torch.cuda.current_stream(g_c.device).cuda_stream)
        _lib.check(rc, "lambda_grad with peer all-reduce")
        return out

    def status(self) -> int:
        """Call number of the last exchange on this device whose wait for a peer ran out (0: none)."""
        return int(self.lib.cnl_peer_allreduce_status())


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
