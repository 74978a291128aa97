"""Batch sharding across the GPUs of one box: contiguous ranges of samples, one process, stream and operator handle
per GPU, no data exchanged between shards (the path has no collective step).

torch.distributed is used for plumbing only -- a start barrier and the max-over-ranks of device-side timings.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_bounds(num_samples: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the samples rank `rank` of `world_size` processes. Ranges are contiguous, disjoint, cover
    0..num_samples and differ in length by at most one (the first num_samples % world_size ranks get the extra one)."""
    if world_size < 1 or not 0 <= rank < world_size or num_samples < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(num_samples, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def all_bounds(num_samples: int, world_size: int) -> List[Tuple[int, int]]:
    return [shard_bounds(num_samples, world_size, r) for r in range(world_size)]


def shard_list(items: Sequence, world_size: int, rank: int) -> Sequence:
    """The slice of a per-sample sequence (images of a variable-shape batch, crop rectangles, flip codes, ...)."""
    b, e = shard_bounds(len(items), world_size, rank)
    return items[b:e]


def max_over_ranks(value: float, device=None) -> float:
    """Largest `value` over all ranks (the job is as slow as its slowest GPU). Identity without a process group."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def aggregate_throughput(images_this_rank: int, elapsed_ms_this_rank: float, device=None) -> float:
    """Whole-job images/s: all images of all ranks over the slowest rank's elapsed time."""
    total = sum_over_ranks(float(images_this_rank), device)
    slowest = max_over_ranks(float(elapsed_ms_this_rank), device)
    return total / (slowest / 1000.0)
