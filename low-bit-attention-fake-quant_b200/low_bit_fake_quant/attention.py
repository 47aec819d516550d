"""Public entry point of the fake-quant attention path (host orchestration).

Drop-in for src/low_bit_fake_quant/attention.py: ``fake_quant_attention``
(:706-806), ``prepare_for_attention`` (:673-703), ``PreprocessCache``
(:647-670), ``FakeQuantArtifacts`` (:77-86), ``reference_attention``
(:809-825) keep their signatures, argument meaning, return types and errors.

What differs is below the API: every device step is a kernel of
``liblbfq.so``. In the P-requant path the quantizers write e4m3 codes
directly in the head-major layouts the attention kernel's TMA descriptors
read (no de-quantised BF16 copies, no NHD->BHSD permutes), the Q-smoothing
correction is one fp32 product ``qm . K_smooth`` whose row max doubles as the
``qm_k`` row-max estimate, and the inverse Q reorder is fused into the
kernel's output store.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib as L
from .attention_triton import fake_quant_attention_fp8, fake_quant_attention_triton, qm_corr
from .config import QuantConfig
from .hadamard import apply_qk_hadamard
from .kmeans import KMeansReorderResult, _gather, apply_kv_permutation, kmeans_reorder_tokens
from .preprocess import group_mean_q, k_channel_mean, smooth_k, smooth_v_per_block
from .quant_triton import (
    fp8_block_dequant,
    fp8_block_quant,
    fp8_per_channel_dequant,
    fp8_per_channel_quant,
    mxfp8_qk_dequant,
    mxfp8_qk_quant,
    mxfp8_v_dequant,
    mxfp8_v_quant,
)


@dataclass
class FakeQuantArtifacts:
    """Side data emitted by :func:`fake_quant_attention` for debugging."""

    qm: Optional[torch.Tensor] = None
    k_mean: Optional[torch.Tensor] = None
    kmeans: Optional[KMeansReorderResult] = None
    q_eff_dtype: Optional[torch.dtype] = None
    p_requant: bool = False
    qk_hadamard: bool = False


@dataclass
class PreprocessCache:
    """Output of :func:`prepare_for_attention`, reusable across configs that
    share the smoothing / k-means / V-smoothing settings recorded here."""

    q_work: torch.Tensor
    k_work: torch.Tensor
    v_work: torch.Tensor
    qm: Optional[torch.Tensor]
    v_alpha: Optional[torch.Tensor]
    q_kmeans: Optional[KMeansReorderResult]
    v_kmeans: Optional[KMeansReorderResult]
    smoothing: str
    q_kmeans_k: Optional[int]
    q_smooth_block_size: int
    v_smooth_mode: str
    v_smooth_block_size: int
    v_kmeans_k: Optional[int]


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


# ---------------------------------------------------------------------------
# preprocess: Q k-means -> K smooth -> Q smooth -> V k-means (+K) -> V smooth
# ---------------------------------------------------------------------------

def _k_smoothing_can_ride_on_the_quantizer(cfg: QuantConfig) -> bool:
    """K smoothing alone, fp8_block K, nothing between the two that needs the smoothed K as a tensor (no score bias,
    no K / V co-permutation, no rotation): the K quantizer subtracts the mean itself."""
    return (cfg.smoothing == "k_only" and cfg.qk_quant == "fp8_block" and cfg.v_kmeans_k is None
            and not cfg.qk_hadamard and cfg.p_requant)


def _preprocess(q, k, v, cfg: QuantConfig, *, head_offset: int = 0, total_heads: int = 0, defer_k_smoothing: bool = False,
                q_labels=None, v_labels=None):
    """The reference's fixed preprocessing order (attention.py:166-239).

    ``defer_k_smoothing`` (only with ``_k_smoothing_can_ride_on_the_quantizer``): K is returned as it came and its
    channel mean as an eighth value, for the quantizer to subtract. ``q_labels`` / ``v_labels`` (B*H, S) replace the
    Lloyd iterations of the corresponding k-means reorder by given cluster assignments (testing aid)."""
    q_work, k_work, v_work = q.contiguous(), k.contiguous(), v.contiguous()
    q_km = v_km = None
    qm = v_alpha = None
    if defer_k_smoothing:
        if cfg.q_kmeans_k is not None:
            q_km = kmeans_reorder_tokens(q_work, n_clusters=cfg.q_kmeans_k, max_iters=cfg.q_kmeans_iters,
                                         seed=cfg.q_kmeans_seed, head_offset=head_offset, total_heads=total_heads,
                                         labels=q_labels)
            q_work = q_km.tensor_reordered
        if cfg.v_smooth_mode == "per_block":
            v_work, v_alpha = smooth_v_per_block(v_work, block_s=cfg.v_smooth_block_size)
        elif cfg.v_smooth_mode != "off":
            raise ValueError(f"unsupported v_smooth_mode: {cfg.v_smooth_mode!r}")
        return q_work, k_work, v_work, None, v_alpha, q_km, None, k_channel_mean(k_work)

    if cfg.q_kmeans_k is not None:
        q_km = kmeans_reorder_tokens(q_work, n_clusters=cfg.q_kmeans_k, max_iters=cfg.q_kmeans_iters,
                                     seed=cfg.q_kmeans_seed, head_offset=head_offset, total_heads=total_heads,
                                     labels=q_labels)
        q_work = q_km.tensor_reordered

    if cfg.smoothing in ("k_only", "full"):
        k_work, _ = smooth_k(k_work)
        if cfg.smoothing == "full":
            q_work, qm = group_mean_q(q_work, block_q=cfg.q_smooth_block_size)
    elif cfg.smoothing != "off":
        raise ValueError(f"unsupported smoothing: {cfg.smoothing!r}")

    if cfg.v_kmeans_k is not None:
        v_km = kmeans_reorder_tokens(v_work, n_clusters=cfg.v_kmeans_k, max_iters=cfg.v_kmeans_iters,
                                     seed=cfg.v_kmeans_seed, head_offset=head_offset, total_heads=total_heads,
                                     labels=v_labels)
        v_work = v_km.tensor_reordered
        k_work = apply_kv_permutation(k_work, v_km.order)      # keep every (K[n], V[n]) pair together

    if cfg.v_smooth_mode == "per_block":
        v_work, v_alpha = smooth_v_per_block(v_work, block_s=cfg.v_smooth_block_size)
    elif cfg.v_smooth_mode != "off":
        raise ValueError(f"unsupported v_smooth_mode: {cfg.v_smooth_mode!r}")

    return q_work, k_work, v_work, qm, v_alpha, q_km, v_km


def _rotated(q_work, k_work, cfg: QuantConfig, head_offset: int = 0, total_heads: int = 0):
    if not cfg.qk_hadamard:
        return q_work, k_work
    return apply_qk_hadamard(q_work, k_work, random_sign=cfg.qk_hadamard_random_sign, seed=cfg.qk_hadamard_seed,
                             head_offset=head_offset, total_heads=total_heads if total_heads > 0 else None,
                             _cross=q_work.shape[1] != k_work.shape[1])


# ---------------------------------------------------------------------------
# path A (p_requant=False): quantise, de-quantise, SDPA  (attention.py:247-321)
# ---------------------------------------------------------------------------

def _quant_dequant_qk(t, cfg: QuantConfig, dtype):
    if cfg.qk_quant == "fp8_block":
        c, s = fp8_block_quant(t, block_s=cfg.fp8_block_size)
        return fp8_block_dequant(c, s, block_s=cfg.fp8_block_size, dtype=dtype)
    if cfg.qk_quant == "mxfp8":
        c, s = mxfp8_qk_quant(t, block_d=cfg.mxfp8_block_size)
        return mxfp8_qk_dequant(c, s, block_d=cfg.mxfp8_block_size, dtype=dtype)
    raise ValueError(f"unsupported qk_quant: {cfg.qk_quant!r}")


def _quant_dequant_v(t, cfg: QuantConfig, dtype):
    if cfg.v_quant == "fp8_channel":
        c, s = fp8_per_channel_quant(t)
        return fp8_per_channel_dequant(c, s, dtype=dtype)
    if cfg.v_quant == "fp8_block":
        c, s = fp8_block_quant(t, block_s=cfg.v_fp8_block_size)
        return fp8_block_dequant(c, s, block_s=cfg.v_fp8_block_size, dtype=dtype)
    if cfg.v_quant == "mxfp8":
        c, s = mxfp8_v_quant(t, block_s=cfg.v_mxfp8_block_size)
        return mxfp8_v_dequant(c, s, block_s=cfg.v_mxfp8_block_size, dtype=dtype)
    raise ValueError(f"unsupported v_quant: {cfg.v_quant!r}")


def _fake_quant_attention_sdpa(q_work, k_work, v_work, qm, v_alpha, cfg: QuantConfig, sm_scale, sdpa_dtype,
                               head_offset: int = 0, total_heads: int = 0):
    """P stays unquantised (upper-bound path). With Q smoothing the score is
    ``Q_deq.K_deq^T + qm.K_smooth^T`` with the second term on the un-quantised K."""
    b, s, h, d = q_work.shape
    q_in, k_in = _rotated(q_work, k_work, cfg, head_offset, total_heads)
    q_deq = _quant_dequant_qk(q_in, cfg, sdpa_dtype)
    k_deq = _quant_dequant_qk(k_in, cfg, sdpa_dtype)
    v_deq = _quant_dequant_v(v_work, cfg, sdpa_dtype)
    if v_alpha is not None:
        bv = cfg.v_smooth_block_size
        if s % bv != 0:
            raise ValueError(f"S={s} not divisible by v_smooth_block_size={bv}")
        v_deq = v_deq + v_alpha.repeat_interleave(bv, dim=1).to(sdpa_dtype)

    to_bh = lambda t: t.permute(0, 2, 1, 3).contiguous()
    if qm is None:
        o = F.scaled_dot_product_attention(to_bh(q_deq), to_bh(k_deq), to_bh(v_deq), scale=sm_scale)
        return o.permute(0, 2, 1, 3).contiguous()

    block_q = cfg.q_smooth_block_size
    chunk = max(block_q, 256)
    qb, kb, vb = to_bh(q_deq), to_bh(k_deq), to_bh(v_deq)
    qmb = to_bh(qm)
    ksb = to_bh(k_work).float()
    out = torch.empty_like(qb)
    group = torch.arange(s, device=q_work.device) // block_q
    for m0 in range(0, s, chunk):
        m1 = min(m0 + chunk, s)
        main = torch.matmul(qb[:, :, m0:m1], kb.transpose(-2, -1)).float() * sm_scale
        corr = torch.matmul(qmb[:, :, group[m0:m1]], ksb.transpose(-2, -1)) * sm_scale
        p = torch.softmax(main + corr, dim=-1).to(sdpa_dtype)
        out[:, :, m0:m1] = torch.matmul(p, vb)
    return out.permute(0, 2, 1, 3).contiguous()


# ---------------------------------------------------------------------------
# path B (p_requant=True): FP8 streaming kernel  (attention.py:505-639)
# ---------------------------------------------------------------------------

def _fake_quant_attention_p_requant(q_work, k_work, v_work, qm, v_alpha, q_kmeans, cfg: QuantConfig,
                                    sm_scale, out_dtype, *, return_stats: bool = False,
                                    out_fp32_exact: bool = False, head_offset: int = 0, total_heads: int = 0,
                                    rowmax_counters=None, k_mean=None, prepared=None,
                                    blasst_tile_predicate: bool = False, blasst_elided=None):
    """Quantise straight into the kernel's layouts and launch it. Returns the
    output in NHD, rows already back in the original Q order.

    ``prepared`` (from ``_prepare_fused``): the codes and scales are there already; ``q_work`` / ``v_work`` are then
    only looked at for their shapes and ``k_work`` is the smoothed K of the score bias (or the input K)."""
    # K / V may have their own length (cross-attention, an extension: the reference's entry takes equal shapes only)
    b, s, h, d = q_work.shape
    s_k = k_work.shape[1]
    sq_pad, s_pad = _round_up(s, 128), _round_up(s_k, 128)
    q_sf = k_sf = None
    if prepared is not None:
        q_codes, q_scale, q_sf = prepared["q"]
        k_codes, k_scale, k_sf = prepared["k"]
    else:
        q_in, k_in = _rotated(q_work, k_work, cfg, head_offset, total_heads)

    if prepared is not None:
        pass
    elif cfg.qk_quant == "fp8_block":
        q_codes, q_scale = fp8_block_quant(q_in, block_s=cfg.fp8_block_size, _layout=L.LAYOUT_BHSD, _s_pad=sq_pad)
        # `k_mean`: K arrives unsmoothed and the quantizer subtracts its channel mean (smooth_k fused in)
        k_codes, k_scale = fp8_block_quant(k_in, block_s=cfg.fp8_block_size, _layout=L.LAYOUT_BHSD, _s_pad=s_pad, _mean=k_mean)
    elif cfg.qk_quant == "mxfp8":
        # codes + UE8M0 scale tiles for the block-scaled MMA (the FP32 scale tensors are by-products here)
        q_sf = torch.empty((b * h * sq_pad * 4,), dtype=torch.uint8, device=q_in.device)
        k_sf = torch.empty((b * h * s_pad * 4,), dtype=torch.uint8, device=q_in.device)
        q_codes, q_scale = mxfp8_qk_quant(q_in, block_d=cfg.mxfp8_block_size, _layout=L.LAYOUT_BHSD, _s_pad=sq_pad, _scale_e8=q_sf)
        k_codes, k_scale = mxfp8_qk_quant(k_in, block_d=cfg.mxfp8_block_size, _layout=L.LAYOUT_BHSD, _s_pad=s_pad, _scale_e8=k_sf)
    else:
        raise ValueError(f"unsupported qk_quant: {cfg.qk_quant!r}")

    v_block = 0
    if prepared is not None:
        v_codes, v_scale = prepared["v"]
        v_block = {"fp8_channel": 0, "fp8_block": cfg.v_fp8_block_size, "mxfp8": cfg.v_mxfp8_block_size}[cfg.v_quant]
    elif cfg.v_quant == "fp8_channel":
        v_codes, v_scale = fp8_per_channel_quant(v_work, _layout=L.LAYOUT_BHDS, _s_pad=s_pad)
    elif cfg.v_quant == "fp8_block":
        v_block = cfg.v_fp8_block_size
        v_codes, v_scale = fp8_block_quant(v_work, block_s=v_block, _layout=L.LAYOUT_BHDS, _s_pad=s_pad)
    elif cfg.v_quant == "mxfp8":
        v_block = cfg.v_mxfp8_block_size
        v_codes, v_scale = mxfp8_v_quant(v_work, block_s=v_block, _layout=L.LAYOUT_BHDS, _s_pad=s_pad)
    else:
        raise ValueError(f"unsupported v_quant: {cfg.v_quant!r}")

    corr = None
    rowmax_est = None
    if cfg.rowmax_mode not in ("online", "qm_k"):
        raise ValueError(f"unsupported rowmax_mode: {cfg.rowmax_mode!r}")
    if cfg.rowmax_mode == "qm_k" and qm is None:
        raise ValueError("rowmax_mode='qm_k' requires smoothing='full' so qm exists")
    if qm is not None:
        want_est = cfg.rowmax_mode == "qm_k"
        corr, rowmax_g = qm_corr(qm, k_work.to(torch.bfloat16), sm_scale=sm_scale, s_pad=s_pad, want_rowmax=want_est)
        if want_est and k_work.dtype != torch.bfloat16:
            # the kernel's bias is formed from the BF16 K, the reference's estimate from K in its own dtype
            # (attention.py:603-608): for FP16 / FP32 inputs the two products differ
            _, rowmax_g = qm_corr(qm, k_work, sm_scale=sm_scale, s_pad=s_pad, want_rowmax=True)
        if want_est:
            rowmax_est = rowmax_g.repeat_interleave(cfg.q_smooth_block_size, dim=2).contiguous()

    p_mode = cfg.p_quant
    if p_mode == "auto":
        p_mode = "mx" if cfg.v_quant == "mxfp8" else "elementwise"
    p_mx_block_n = cfg.p_mx_block_n if cfg.p_mx_block_n > 0 else cfg.v_mxfp8_block_size

    return fake_quant_attention_fp8(
        q_codes, k_codes, v_codes,
        seq_q=s, seq_k=s_k,
        q_scale=q_scale, k_scale=k_scale,
        qk_block=cfg.fp8_block_size if cfg.qk_quant == "fp8_block" else cfg.mxfp8_block_size,
        q_scale_e8=q_sf, k_scale_e8=k_sf,
        v_kind=cfg.v_quant, v_scale=v_scale, v_block=v_block,
        sm_scale=float(sm_scale), p_max_offset=int(cfg.p_max_offset),
        block_m=cfg.p_requant_block_m, block_n=cfg.p_requant_block_n,
        v_alpha=v_alpha, v_smooth_block=cfg.v_smooth_block_size if v_alpha is not None else 0,
        qm_corr=corr, q_smooth_block=cfg.q_smooth_block_size if qm is not None else 0,
        p_quant_mode=p_mode, p_mx_block_n=p_mx_block_n,
        rowmax_est_bhs=rowmax_est,
        blasst_lambda=cfg.blasst_lambda, blasst_fill_mode=cfg.blasst_fill,
        blasst_fill_alpha=cfg.blasst_fill_alpha, blasst_uta_bins=cfg.blasst_uta_bins,
        return_blasst_stats=return_stats,
        blasst_tile_predicate=blasst_tile_predicate, blasst_elided=blasst_elided,
        out_dtype=torch.float32 if out_fp32_exact else out_dtype, out_nhd=True,
        out_row_index=q_kmeans.order if q_kmeans is not None else None,
        out_fp32_exact=out_fp32_exact,
        rowmax_counters=rowmax_counters,
    )


_SIDE_STREAMS: dict = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """One extra stream per device for work that is independent of the current stream's (kept for the process)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    st = _SIDE_STREAMS.get(key)
    if st is None:
        st = _SIDE_STREAMS[key] = torch.cuda.Stream(device)
    return st


def _prepare_fused(q, k, v, cfg: QuantConfig, *, head_offset: int = 0, total_heads: int = 0, q_labels=None, v_labels=None):
    """Preprocessing (attention.py:166-239 of the reference) and quantisation (:531-570) of all three tensors with one
    fused pass per tensor (``prepare.prep_fused``): the k-means orders and the K channel mean are found first, then
    each tensor is gathered, smoothed, rotated and quantised straight into the kernel's layout. Returns the dictionary
    ``_fake_quant_attention_p_requant`` takes as ``prepared`` (plus qm, v_alpha, the Q reorder and the smoothed K), or
    ``None`` when some block size combination is not served by the fused kernel (the caller then runs the separate
    kernels). Every value equals the separate kernels' bit for bit."""
    from .kmeans import kmeans_labels, order_from_labels
    from .prepare import group_rows, hadamard_signs, prep_fused

    b, s, h, d = q.shape
    s_k = k.shape[1]
    if cfg.qk_quant not in ("fp8_block", "mxfp8") or cfg.v_quant not in ("fp8_channel", "fp8_block", "mxfp8"):
        return None
    if cfg.smoothing not in ("off", "k_only", "full") or cfg.v_smooth_mode not in ("off", "per_block"):
        return None
    full = cfg.smoothing == "full"
    qk_kind = "fp8_block" if cfg.qk_quant == "fp8_block" else "mxfp8_qk"
    qk_block = cfg.fp8_block_size if cfg.qk_quant == "fp8_block" else cfg.mxfp8_block_size
    v_kind = {"fp8_channel": "fp8_channel", "fp8_block": "fp8_block", "mxfp8": "mxfp8_v"}[cfg.v_quant]
    v_block = {"fp8_channel": 0, "fp8_block": cfg.v_fp8_block_size, "mxfp8": cfg.v_mxfp8_block_size}[cfg.v_quant]
    q_sb = cfg.q_smooth_block_size if full else 0
    v_sb = cfg.v_smooth_block_size if cfg.v_smooth_mode == "per_block" else 0
    for kind, sb, blk, seq in ((qk_kind, q_sb, qk_block, s), (qk_kind, 0, qk_block, s_k), (v_kind, v_sb, v_block, s_k)):
        if (sb > 0 and seq % sb != 0) or (kind in ("fp8_block", "mxfp8_v") and (blk <= 0 or seq % blk != 0)):
            return None                                   # the separate kernels raise the reference's errors for these
        if kind == "mxfp8_qk" and (blk <= 0 or d % blk != 0 or blk % 8 != 0 or (blk & (blk - 1)) != 0 or d // blk > 4):
            return None
        if group_rows(kind, smooth_block=sb, scale_block=blk, seq=seq, dim=d, dtype=q.dtype) <= 0:
            return None
    if s % 16 != 0 or s_k % 16 != 0:
        return None
    sq_pad, s_pad = _round_up(s, 128), _round_up(s_k, 128)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()

    q_km = None
    q_order = v_order = None
    if cfg.v_kmeans_k is not None and (cfg.v_kmeans_k <= 0 or cfg.v_kmeans_k > s_k):
        return None
    side = None
    if cfg.q_kmeans_k is not None and cfg.v_kmeans_k is not None and q_labels is None and v_labels is None:
        # the two clusterings are independent, and a Lloyd iteration is a chain of short kernels (assignment, sort,
        # segment means) none of which fills the GPU to its end: V's runs on a second stream next to Q's
        cur = torch.cuda.current_stream(q.device)
        side = _side_stream(q.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            lab_v = kmeans_labels(v, n_clusters=cfg.v_kmeans_k, max_iters=cfg.v_kmeans_iters, seed=cfg.v_kmeans_seed,
                                  head_offset=head_offset, total_heads=total_heads)
            v_order, v_inv = order_from_labels(lab_v, cfg.v_kmeans_k)
        for t in (lab_v, v_order, v_inv):
            t.record_stream(cur)
    if cfg.q_kmeans_k is not None:
        if cfg.q_kmeans_k <= 0 or cfg.q_kmeans_k > s:
            return None
        lab = q_labels if q_labels is not None else kmeans_labels(
            q, n_clusters=cfg.q_kmeans_k, max_iters=cfg.q_kmeans_iters, seed=cfg.q_kmeans_seed, head_offset=head_offset,
            total_heads=total_heads)
        q_order, q_inv = order_from_labels(lab, cfg.q_kmeans_k)
        q_km = KMeansReorderResult(tensor_reordered=None, order=q_order, inverse_order=q_inv, labels=lab.to(torch.int64))
    k_mean = k_channel_mean(k) if cfg.smoothing in ("k_only", "full") else None       # over K in its own order
    if side is None and cfg.v_kmeans_k is not None:
        lab = v_labels if v_labels is not None else kmeans_labels(
            v, n_clusters=cfg.v_kmeans_k, max_iters=cfg.v_kmeans_iters, seed=cfg.v_kmeans_seed, head_offset=head_offset,
            total_heads=total_heads)
        v_order, _ = order_from_labels(lab, cfg.v_kmeans_k)
    signs = None
    if cfg.qk_hadamard and cfg.qk_hadamard_random_sign:
        signs = hadamard_signs(h, d, cfg.qk_hadamard_seed, q.device, head_offset=head_offset,
                               total_heads=total_heads if total_heads > 0 else None)
    mx = cfg.qk_quant == "mxfp8"
    qc, qs, qm, q_sf, _ = prep_fused(q, kind=qk_kind, scale_block=qk_block, order=q_order, smooth_block=q_sb,
                                     hadamard=cfg.qk_hadamard, signs=signs, layout=L.LAYOUT_BHSD, s_pad=sq_pad, want_scale_e8=mx)
    if side is not None:
        torch.cuda.current_stream(q.device).wait_stream(side)       # K and V follow V's order; Q did not need it
    kc, ks, _, k_sf, k_smooth = prep_fused(k, kind=qk_kind, scale_block=qk_block, order=v_order, chan_mean=k_mean,
                                           hadamard=cfg.qk_hadamard, signs=signs, layout=L.LAYOUT_BHSD, s_pad=s_pad,
                                           want_scale_e8=mx, want_prepared=full)
    vc, vs, v_alpha, _, _ = prep_fused(v, kind=v_kind, scale_block=v_block, order=v_order, smooth_block=v_sb,
                                       layout=L.LAYOUT_BHDS, s_pad=s_pad)
    return {"q": (qc, qs, q_sf), "k": (kc, ks, k_sf), "v": (vc, vs), "qm": qm, "v_alpha": v_alpha, "q_kmeans": q_km,
            "k_smooth": k_smooth if full else k}


# ---------------------------------------------------------------------------
# public entry points
# ---------------------------------------------------------------------------

def prepare_for_attention(q, k, v, cfg: QuantConfig) -> PreprocessCache:
    """Run k-means + Q/K smoothing + V smoothing without any quantization."""
    if q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q/k/v shapes must match")
    if q.ndim != 4 or not q.is_cuda:
        raise ValueError("q/k/v must be 4-D NHD on CUDA")
    q_work, k_work, v_work, qm, v_alpha, q_km, v_km = _preprocess(q, k, v, cfg)
    return PreprocessCache(
        q_work=q_work, k_work=k_work, v_work=v_work, qm=qm, v_alpha=v_alpha, q_kmeans=q_km, v_kmeans=v_km,
        smoothing=cfg.smoothing, q_kmeans_k=cfg.q_kmeans_k, q_smooth_block_size=cfg.q_smooth_block_size,
        v_smooth_mode=cfg.v_smooth_mode, v_smooth_block_size=cfg.v_smooth_block_size, v_kmeans_k=cfg.v_kmeans_k,
    )


def _fake_quant_attention_p_requant_reference_operands(q_work, k_work, v_work, qm, v_alpha, q_kmeans, cfg: QuantConfig,
                                                       sm_scale, out_dtype, *, out_fp32_exact: bool = False,
                                                       head_offset: int = 0, total_heads: int = 0):
    """Path B with the operands the reference itself builds (attention.py:505-639): Q / K de-quantised to BF16,
    V as BF16 code values with its per-channel scale (or de-quantised for mxfp8), handed to the direct-launch
    entry. Q.K^T and P.V then run as BF16 MMAs, i.e. in the reference's numerics."""
    q_in, k_in = _rotated(q_work, k_work, cfg, head_offset, total_heads)
    q_deq = _quant_dequant_qk(q_in, cfg, torch.bfloat16)
    k_deq = _quant_dequant_qk(k_in, cfg, torch.bfloat16)
    b, s, h, d = q_work.shape
    if cfg.v_quant == "fp8_channel":
        codes, v_scale = fp8_per_channel_quant(v_work)
        v_bf = codes.to(torch.bfloat16)                       # code values, exact in BF16
    elif cfg.v_quant == "mxfp8":
        v_bf = _quant_dequant_v(v_work, cfg, torch.bfloat16)  # codes x 2^e, exact in BF16
        v_scale = torch.ones((b, h, d), dtype=torch.float32, device=v_work.device)
    elif cfg.v_quant == "fp8_block":
        codes, v_block_scale = fp8_block_quant(v_work, block_s=cfg.v_fp8_block_size)
        v_bf = codes.to(torch.bfloat16)
        v_scale = torch.ones((b, h, d), dtype=torch.float32, device=v_work.device)
    else:
        raise ValueError(f"unsupported v_quant: {cfg.v_quant!r}")
    if cfg.rowmax_mode not in ("online", "qm_k"):
        raise ValueError(f"unsupported rowmax_mode: {cfg.rowmax_mode!r}")
    if cfg.rowmax_mode == "qm_k" and qm is None:
        raise ValueError("rowmax_mode='qm_k' requires smoothing='full' so qm exists")
    to_bh = lambda t: t.permute(0, 2, 1, 3).contiguous()
    rowmax_est = corr = None
    block_kw = {}
    if cfg.v_quant == "fp8_block":
        block_kw.update(v_block_scale_bsh=v_block_scale.float().contiguous(), v_block_size=cfg.v_fp8_block_size)
    if cfg.blasst_lambda is not None:
        block_kw.update(blasst_lambda=cfg.blasst_lambda, blasst_fill_mode=cfg.blasst_fill,
                        blasst_fill_alpha=cfg.blasst_fill_alpha, blasst_uta_bins=cfg.blasst_uta_bins)
    if qm is not None:
        # one product serves the score bias and the row-max estimate; the launcher takes it instead of forming it again
        want_est = cfg.rowmax_mode == "qm_k"
        corr, rowmax_g = qm_corr(qm, k_work.to(torch.bfloat16), sm_scale=sm_scale, s_pad=_round_up(k_work.shape[1], 128),
                                 want_rowmax=want_est)
        if want_est and k_work.dtype != torch.bfloat16:       # the estimate comes from K in its own dtype
            _, rowmax_g = qm_corr(qm, k_work, sm_scale=sm_scale, s_pad=_round_up(k_work.shape[1], 128), want_rowmax=True)
        if want_est:
            rowmax_est = rowmax_g.repeat_interleave(cfg.q_smooth_block_size, dim=2).contiguous()
    p_mode = cfg.p_quant
    if p_mode == "auto":
        p_mode = "mx" if cfg.v_quant == "mxfp8" else "elementwise"
    p_mx_block_n = cfg.p_mx_block_n if cfg.p_mx_block_n > 0 else cfg.v_mxfp8_block_size
    o = fake_quant_attention_triton(
        to_bh(q_deq), to_bh(k_deq), to_bh(v_bf), v_scale,
        sm_scale=float(sm_scale), p_max_offset=int(cfg.p_max_offset),
        block_m=cfg.p_requant_block_m, block_n=cfg.p_requant_block_n,
        v_alpha=v_alpha, v_smooth_block=cfg.v_smooth_block_size if v_alpha is not None else 0,
        k_smooth_bhsd=to_bh(k_work.to(torch.bfloat16)) if qm is not None else None,
        qm_bhgd=qm.float().contiguous() if qm is not None else None,      # (B, G, H, D), as group_mean_q returns it
        q_smooth_block=cfg.q_smooth_block_size if qm is not None else 0,
        p_quant_mode=p_mode, p_mx_block_n=p_mx_block_n, rowmax_est_bhs=rowmax_est, _out_fp32=out_fp32_exact, _corr=corr,
        **block_kw)
    o = o.permute(0, 2, 1, 3).contiguous()                    # (B, S, H, D)
    o = o if out_fp32_exact else o.to(out_dtype)
    if q_kmeans is not None:
        o = _gather(o, q_kmeans.inverse_order)
    return o


def fake_quant_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cfg: Optional[QuantConfig] = None,
    *,
    sm_scale: Optional[float] = None,
    return_artifacts: bool = False,
    preprocess_cache: Optional[PreprocessCache] = None,
    _debug_fp32: bool = False,
    _cross: bool = False,
    _head_offset: int = 0,
    _total_heads: int = 0,
    _reference_operands: bool = False,
    _q_labels: Optional[torch.Tensor] = None,
    _v_labels: Optional[torch.Tensor] = None,
    _blasst_tile_predicate: bool = False,
    _blasst_elided: Optional[torch.Tensor] = None,
):
    """Fake-quant attention with FP8/MXFP8 Q/K/V (and optional P requant).

    ``q, k, v``: (B, S, H, D), D in {64, 128}, BF16/FP16/FP32 on CUDA.
    Returns the (B, S, H, D) output in ``q``'s dtype (and the artifacts). The launches are asynchronous; a kernel
    that gives up one of its bounded waits (which only a stalled device can cause) reports it through a status word
    that is examined on the next call on that device and by ``attention_triton.raise_if_device_error()``: call the
    latter before trusting a result if such a stall is a possibility.
    ``_debug_fp32`` (testing aid) returns the kernel's FP32 result without the
    BF16 rounding of the store. ``_head_offset`` / ``_total_heads`` tell a heads
    shard where it sits in the unsharded problem (Hadamard signs and k-means
    seeding are indexed by global head), so that sharded == unsharded.
    ``_reference_operands`` runs path B on the reference's own BF16 operands
    (BF16 MMAs) instead of the FP8 codes: the reference's numerics, at BF16 speed.
    ``_q_labels`` / ``_v_labels`` (testing aid) give the k-means reorders their cluster assignments.
    ``_blasst_tile_predicate`` (extension): BLASST drops a key block only when every row of a 128-row tile finds it
    under the threshold, and then for the whole tile -- the predicate of the reference's simulator
    (blasst_skip.py:573-585) instead of the kernel's row-by-row one; zero fill. ``_blasst_elided``: one int64 zero on
    the device that receives the number of (tile, key block) pairs the kernel did no work for.
    """
    if cfg is None:
        cfg = QuantConfig()
    if _cross:
        # extension (hook.fake_quant_cross_attention): K / V of their own length, streaming path only
        ok = (q.ndim == k.ndim == 4 and k.shape == v.shape and q.shape[0] == k.shape[0] and q.shape[2:] == k.shape[2:])
        if not ok:
            raise ValueError(f"cross-attention wants q (B,Sq,H,D) and k, v (B,Sk,H,D); got {tuple(q.shape)}, "
                             f"{tuple(k.shape)}, {tuple(v.shape)}")
        if not cfg.p_requant:
            raise ValueError("cross-attention is served by the streaming kernel: requires cfg.p_requant=True")
    elif q.shape != k.shape or q.shape != v.shape:
        raise ValueError(f"q/k/v shapes must match; got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if q.ndim != 4:
        raise ValueError(f"q/k/v must be 4-D (B,S,H,D); got {q.shape}")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("q/k/v must live on CUDA")
    out_dtype = q.dtype
    if out_dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError(f"unsupported dtype {out_dtype}")
    sdpa_dtype = torch.float16 if out_dtype == torch.float16 else torch.bfloat16
    d = q.shape[-1]
    if d not in (64, 128):
        # every operator under this entry is built for these two head dimensions (quant_triton.py:21-22 of the
        # reference refuses the others at its first quantizer; here nothing is launched at all)
        raise ValueError(f"tensor.shape[-1] must be 64 or 128; got {d}")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    if cfg.blasst_lambda is not None and not cfg.p_requant:
        raise ValueError("BLASST skip/fill requires cfg.p_requant=True")

    # everything in front of the streaming kernel as one fused pass per tensor, when nothing asks for the
    # intermediate tensors (a cache, the artifacts, the reference's own operands) and the kernel takes the codes
    if (preprocess_cache is None and cfg.p_requant and not _reference_operands and not return_artifacts
            and not (L.flags() & L.FLAG_UNFUSED_PREPROCESS)):
        prep = _prepare_fused(q, k, v, cfg, head_offset=_head_offset, total_heads=_total_heads, q_labels=_q_labels,
                              v_labels=_v_labels)
        if prep is not None:
            return _fake_quant_attention_p_requant(
                q, prep["k_smooth"], v, prep["qm"], prep["v_alpha"], prep["q_kmeans"], cfg, sm_scale, out_dtype,
                out_fp32_exact=_debug_fp32, head_offset=_head_offset, total_heads=_total_heads, prepared=prep,
                blasst_tile_predicate=_blasst_tile_predicate, blasst_elided=_blasst_elided)

    if preprocess_cache is not None:
        pc = preprocess_cache
        same = (pc.smoothing == cfg.smoothing and pc.q_kmeans_k == cfg.q_kmeans_k
                and pc.q_smooth_block_size == cfg.q_smooth_block_size and pc.v_smooth_mode == cfg.v_smooth_mode
                and pc.v_smooth_block_size == cfg.v_smooth_block_size and pc.v_kmeans_k == cfg.v_kmeans_k)
        if not same:
            raise ValueError("preprocess_cache does not match cfg's smoothing/kmeans/v_smooth settings")
        q_work, k_work, v_work, qm, v_alpha, q_km = pc.q_work, pc.k_work, pc.v_work, pc.qm, pc.v_alpha, pc.q_kmeans
        k_mean = None
    else:
        # where nothing else needs the smoothed K, it is never stored: the K quantizer subtracts the mean
        defer = _k_smoothing_can_ride_on_the_quantizer(cfg) and not _reference_operands
        pre = _preprocess(q, k, v, cfg, head_offset=_head_offset, total_heads=_total_heads, defer_k_smoothing=defer,
                          q_labels=_q_labels, v_labels=_v_labels)
        q_work, k_work, v_work, qm, v_alpha, q_km = pre[:6]
        k_mean = pre[7] if defer else None

    # (mxfp8 Q / K codes reach the kernel with the accumulator in tensor memory as exact BF16 operands: the library
    # converts them itself, lbfq_attention_fwd)
    if cfg.p_requant and _reference_operands:
        o = _fake_quant_attention_p_requant_reference_operands(
            q_work, k_work, v_work, qm, v_alpha, q_km, cfg, sm_scale, out_dtype, out_fp32_exact=_debug_fp32,
            head_offset=_head_offset, total_heads=_total_heads)
    elif cfg.p_requant:
        # the kernel scatters its rows through q_km.order: no separate inverse gather
        o = _fake_quant_attention_p_requant(q_work, k_work, v_work, qm, v_alpha, q_km, cfg, sm_scale, out_dtype,
                                            out_fp32_exact=_debug_fp32, head_offset=_head_offset,
                                            total_heads=_total_heads, k_mean=k_mean,
                                            blasst_tile_predicate=_blasst_tile_predicate,
                                            blasst_elided=_blasst_elided)
    else:
        o = _fake_quant_attention_sdpa(q_work, k_work, v_work, qm, v_alpha, cfg, sm_scale, sdpa_dtype,
                                       _head_offset, _total_heads)
        o = o.float() if _debug_fp32 else o.to(out_dtype)
        if q_km is not None:
            o = _gather(o, q_km.inverse_order)

    if return_artifacts:
        return o, FakeQuantArtifacts(qm=qm, kmeans=q_km, q_eff_dtype=sdpa_dtype, p_requant=cfg.p_requant,
                                     qk_hadamard=cfg.qk_hadamard)
    return o


def reference_attention(q, k, v, *, sm_scale: Optional[float] = None) -> torch.Tensor:
    """BF16 SDPA on the raw inputs: the accuracy baseline."""
    if q.ndim != 4:
        raise ValueError(f"q/k/v must be (B,S,H,D); got {q.shape}")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    o = F.scaled_dot_product_attention(q.permute(0, 2, 1, 3).contiguous(), k.permute(0, 2, 1, 3).contiguous(),
                                       v.permute(0, 2, 1, 3).contiguous(), scale=sm_scale)
    return o.permute(0, 2, 1, 3).contiguous()


__all__ = ["FakeQuantArtifacts", "PreprocessCache", "fake_quant_attention", "prepare_for_attention",
           "reference_attention"]
