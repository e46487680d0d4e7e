"""Batch sharding across the GPUs of one box.  The forward pass of a convolution needs no
exchange between images, so each rank (one process per GPU) takes a contiguous slice of the
batch, holds its own copy of the transformed filters and keeps its outputs; the only
cross-rank traffic is the host-side barrier and the max-over-ranks of the elapsed time that
the benchmark reports.  The reference has no multi-GPU code at all."""
from __future__ import annotations

from typing import List, Tuple


def shard_bounds(total: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of ``rank``'s slice of ``total`` items; the remainder goes to the first ranks."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if total < 0:
        raise ValueError("total must be non-negative")
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def all_shards(total: int, world: int) -> List[Tuple[int, int]]:
    return [shard_bounds(total, world, r) for r in range(world)]


def aggregate_throughput(units_per_rank, seconds_per_rank) -> float:
    """Whole-job throughput: all units processed / the slowest rank's time."""
    slowest = max(seconds_per_rank)
    if slowest <= 0:
        raise ValueError("elapsed time must be positive")
    return float(sum(units_per_rank)) / slowest


def max_over_ranks(value: float, group=None) -> float:
    """MAX all-reduce of a host float over the process group (gloo or nccl); identity when
    torch.distributed is not initialised."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sum_over_ranks(value: float, group=None) -> float:
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())
