"""Data-parallel plumbing of the layer: the batch is sharded over ranks (one process per GPU) and the only
collective is a sum all-reduce of the learned-scalar gradients.  Uses torch.distributed (NCCL on GPUs, gloo in
CPU tests); images never cross ranks."""
from __future__ import annotations

from typing import Tuple

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
