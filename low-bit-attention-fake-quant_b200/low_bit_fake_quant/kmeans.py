"""Token k-means reorder (CUDA, sm_100a).

API of src/low_bit_fake_quant/kmeans.py:26-135. The reference calls the
third-party ``flash_kmeans.batch_kmeans_Euclid``; here Lloyd's iterations,
the stable label sort and the row gather are kernels of ``liblbfq.so``
(csrc/kmeans.cu, csrc/preprocess.cu). Unlike the reference this does not
reseed torch's global RNG: the centroid seeding is a hash of
``(seed, global slab index, cluster)``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib as L


@dataclass
class KMeansReorderResult:
    tensor_reordered: torch.Tensor
    order: torch.Tensor
    inverse_order: torch.Tensor
    labels: torch.Tensor

    @property
    def q_reordered(self) -> torch.Tensor:  # pragma: no cover - trivial
        return self.tensor_reordered

    @property
    def v_reordered(self) -> torch.Tensor:  # pragma: no cover - trivial
        return self.tensor_reordered


def kmeans_labels(t: torch.Tensor, *, n_clusters: int, max_iters: int = 10, seed: int = 0,
                  head_offset: int = 0, total_heads: int = 0) -> torch.Tensor:
    """int32 labels (B*H, S) of the last Lloyd assignment. ``head_offset`` / ``total_heads``
    place a heads shard inside the unsharded problem (they only enter the seeding hash)."""
    b, s, h, d = t.shape
    t = t.contiguous()
    labels = torch.empty((b * h, s), dtype=torch.int32, device=t.device)
    with torch.cuda.device(t.device):
        nbytes = L.lib().lbfq_kmeans_scratch_bytes(b, s, h, d, n_clusters)
        scratch = torch.empty((nbytes,), dtype=torch.uint8, device=t.device)
        status = L.status_for(t.device)
        L.check(L.lib().lbfq_kmeans_labels(t.data_ptr(), L.dtype_code(t.dtype), b, s, h, d, n_clusters,
                                           max_iters, seed, head_offset, total_heads, labels.data_ptr(), scratch.data_ptr(),
                                           status.data_ptr(), L.stream_ptr(t.device)))
        L.fetch_status(t.device)
    return labels


def order_from_labels(labels: torch.Tensor, n_clusters: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Stable argsort of ``labels`` (BH, S) and its inverse, both int64."""
    bh, s = labels.shape
    lab = labels.to(torch.int32).contiguous()
    order = torch.empty((bh, s), dtype=torch.int64, device=labels.device)
    inverse = torch.empty_like(order)
    with torch.cuda.device(labels.device):
        L.check(L.lib().lbfq_label_order(lab.data_ptr(), bh, s, n_clusters, order.data_ptr(),
                                         inverse.data_ptr(), L.stream_ptr(labels.device)))
    return order, inverse


def _gather(t: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    b, s, h, d = t.shape
    t = t.contiguous()
    out = torch.empty_like(t)
    index = index.contiguous()
    with torch.cuda.device(t.device):
        L.check(L.lib().lbfq_gather_rows(t.data_ptr(), L.dtype_code(t.dtype), b, s, h, d, index.data_ptr(),
                                         out.data_ptr(), L.stream_ptr(t.device)))
    return out


def kmeans_reorder_tokens(
    t: torch.Tensor,
    *,
    n_clusters: int,
    max_iters: int = 10,
    seed: int = 0,
    chunk_tokens: int = 4096,  # kept for signature compatibility; unused
    labels: torch.Tensor | None = None,
    head_offset: int = 0,
    total_heads: int = 0,
) -> KMeansReorderResult:
    """Cluster tokens of ``t`` (B, S, H, D) per (B, H) and reorder them by cluster.

    ``labels`` (extension) injects precomputed assignments instead of running
    Lloyd's iterations.
    """
    del chunk_tokens
    if t.ndim != 4 or not t.is_cuda:
        raise ValueError(f"t must be 4-D NHD on CUDA; got {tuple(t.shape)} on {t.device}")
    b, s, h, d = t.shape
    if n_clusters <= 0 or n_clusters > s:
        raise ValueError(f"n_clusters must be in [1, S]; got {n_clusters} for S={s}")
    if labels is None:
        labels = kmeans_labels(t, n_clusters=n_clusters, max_iters=max_iters, seed=seed, head_offset=head_offset,
                               total_heads=total_heads)
    order, inverse = order_from_labels(labels, n_clusters)
    return KMeansReorderResult(
        tensor_reordered=_gather(t, order),
        order=order,
        inverse_order=inverse,
        labels=labels.to(torch.int64),
    )


def q_kmeans_reorder(q: torch.Tensor, *, n_clusters: int = 32, max_iters: int = 10, seed: int = 0,
                     chunk_tokens: int = 4096) -> KMeansReorderResult:
    """Cluster Q tokens per (B, H) and reorder them; attention output rows must be
    inverse-permuted to restore the original order."""
    return kmeans_reorder_tokens(q, n_clusters=n_clusters, max_iters=max_iters, seed=seed, chunk_tokens=chunk_tokens)


def v_kmeans_reorder(v: torch.Tensor, *, n_clusters: int = 32, max_iters: int = 10, seed: int = 0) -> KMeansReorderResult:
    """Cluster V tokens per (B, H) and reorder; K must be co-permuted with ``order``."""
    return kmeans_reorder_tokens(v, n_clusters=n_clusters, max_iters=max_iters, seed=seed)


def apply_kv_permutation(t: torch.Tensor, order: torch.Tensor) -> torch.Tensor:
    """Apply a (B*H, S) permutation along S of a (B, S, H, D) tensor."""
    if t.ndim != 4:
        raise ValueError(f"t must be (B,S,H,D); got {tuple(t.shape)}")
    return _gather(t, order)
