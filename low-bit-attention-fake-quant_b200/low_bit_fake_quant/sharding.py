"""Batch x heads sharding of the attention path across the GPUs of one box.

Every (b, h) slab of the path is independent end to end (k-means, smoothing,
every scale tensor, the attention grid and the inverse reorder are all indexed
by (b, h)), so a multi-GPU run is a partition of the slabs with no collective
on the data path. The only things that must see the GLOBAL head index are the
Hadamard sign table and the k-means seeding hash; both take an offset.
"""

from __future__ import annotations

from typing import List, Tuple


def slab_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) of ``total`` slabs owned by ``rank``; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def all_ranges(total: int, world: int) -> List[Tuple[int, int]]:
    return [slab_range(total, world, r) for r in range(world)]


def head_shard(q, k, v, world: int, rank: int):
    """Slice (B, S, H, D) tensors to this rank's heads; returns the tensors and the head offset."""
    lo, hi = slab_range(q.shape[2], world, rank)
    return q[:, :, lo:hi].contiguous(), k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous(), lo
