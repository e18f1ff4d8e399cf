"""Batch sharding of the BTP path over the GPUs of one box.

Every (batch, head) sequence is independent, so N ranks each take a contiguous
slice of the batch and nothing is exchanged on the data path.  The only
collectives are the ones a checker or a benchmark needs afterwards: the maximum
of a timing over ranks and global error norms.  They run on whatever backend the
process group has (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist


def batch_shard(global_batch: int, rank: int, world: int) -> tuple[int, int]:
    """[start, stop) of `rank`'s slice; slices differ by at most one entry and cover the batch exactly."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if global_batch < 0:
        raise ValueError("global_batch must be >= 0")
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def _world(group=None) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def max_over_ranks(values, device=None, group=None) -> list[float]:
    """Element-wise maximum of a few floats over all ranks (timings are reported as the slowest rank)."""
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    if _world(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.tolist()


def sum_over_ranks(values, device=None, group=None) -> list[float]:
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    if _world(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t.tolist()


def global_rel_l2(got: torch.Tensor, want: torch.Tensor, group=None) -> float:
    """||got - want|| / ||want|| over the shards of all ranks (each rank passes its own shard)."""
    g = got.detach().double()
    w = want.detach().double()
    num, den = sum_over_ranks([(g - w).square().sum().item(), w.square().sum().item()], device=got.device, group=group)
    return math.sqrt(num) / math.sqrt(den) if den > 0 else math.sqrt(num)
