"""Batch x heads sharding of the attention path across the GPUs of one box.

Every (b, h) slab of the path is independent end to end (k-means, smoothing,
every scale tensor, the attention grid and the inverse reorder are all indexed
by (b, h)), so a multi-GPU run is a partition of the slabs with no collective
on the data path. The only things that must see the GLOBAL head index are the
Hadamard sign table and the k-means seeding hash; both take an offset.

``attention_on_shard`` is what a rank of such a run calls (``bench.py`` does,
for its strong-scaling figure); ``gather_heads`` assembles the full output
where a caller wants it in one place (one all-gather, outside the data path).
"""

from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch


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


def attention_on_shard(q, k, v, cfg, *, world: int, rank: int, attention: Optional[Callable] = None, **kwargs):
    """This rank's share of ONE attention problem: heads ``slab_range(H, world, rank)`` of (B, S, H, D) tensors.

    ``q, k, v`` are either the full tensors (sliced here) or already this rank's heads when ``sliced=True`` is passed.
    The shard is told where it sits in the full problem, so that the concatenation of all ranks' results along the
    heads axis equals the unsharded call bit for bit. Returns ``(out_local, head_offset)``. ``attention`` defaults
    to this package's ``fake_quant_attention`` (tests inject a stand-in that takes the same two keywords)."""
    total_heads = kwargs.pop("total_heads", None)
    if kwargs.pop("sliced", False):
        if total_heads is None:
            raise ValueError("sliced=True needs total_heads")
        lo, hi = slab_range(total_heads, world, rank)
        if q.shape[2] != hi - lo:
            raise ValueError(f"rank {rank} of {world} owns {hi - lo} of {total_heads} heads; got {q.shape[2]}")
        qs, ks, vs = q, k, v
    else:
        total_heads = q.shape[2]
        qs, ks, vs, lo = head_shard(q, k, v, world, rank)
    if attention is None:
        from .attention import fake_quant_attention as attention
    return attention(qs, ks, vs, cfg, _head_offset=lo, _total_heads=total_heads, **kwargs), lo


def gather_heads(out_local: torch.Tensor, total_heads: int, *, group=None) -> torch.Tensor:
    """All ranks' (B, S, h_r, D) results concatenated along heads into (B, S, total_heads, D), on every rank.

    One ``all_gather`` over the process group (NCCL over NVLink for CUDA tensors, gloo on CPU); uneven shards are
    padded to the largest one for the collective and trimmed afterwards. Not part of the attention path itself:
    callers that keep working head-parallel never need it."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    ranges = all_ranges(total_heads, world)
    h_max = max(hi - lo for lo, hi in ranges)
    b, s, h_r, d = out_local.shape
    padded = out_local
    if h_r < h_max:
        padded = out_local.new_zeros((b, s, h_max, d))
        padded[:, :, :h_r] = out_local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p[:, :, : hi - lo] for p, (lo, hi) in zip(parts, ranges)], dim=2)
