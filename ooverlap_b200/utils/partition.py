"""Partition arithmetic shared by the collectives.

Capability parity: src/comm/utils/collective_utils.h:34-61 of the reference
(uneven partitions give ``base + 1`` elements to the first ``count % world``
ranks).
"""
from __future__ import annotations


def partition(count: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open element range ``[begin, end)`` owned by ``rank``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world {world}")
    if count < 0:
        raise ValueError("negative count")
    base, rem = divmod(count, world)
    begin = base * rank + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def partition_sizes(count: int, world: int) -> list[int]:
    return [partition(count, world, r)[1] - partition(count, world, r)[0] for r in range(world)]


def max_shard(count: int, world: int) -> int:
    return -(-count // world)


def bus_bandwidth_gbs(collective: str, world: int, nbytes: int, seconds: float) -> float:
    """Bus bandwidth in GB/s with the reference's definition (tool/bandwidth.py:263-275):
    all-reduce ``2(n-1)/n * S / t``, reduce-scatter and all-gather ``(n-1)/n * S / t``
    where S is the full message size."""
    if seconds <= 0:
        return 0.0
    n = world
    if collective in ("all_reduce", "allreduce"):
        factor = 2.0 * (n - 1) / n
    elif collective in ("reduce_scatter", "all_gather", "reducescatter", "allgather"):
        factor = (n - 1) / n
    else:
        raise ValueError(collective)
    return factor * nbytes / seconds / 1e9
