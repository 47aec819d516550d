"""``prepare_qkv``: preprocess + quantise, returning codes and scales.

Same dataclass and function as src/low_bit_fake_quant/pipeline.py:19-110 --
the public surface on which the quantizers' codes and scales are observable.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .attention_triton import qm_corr
from .config import QuantConfig
from .hadamard import apply_qk_hadamard
from .kmeans import KMeansReorderResult, q_kmeans_reorder
from .preprocess import group_mean_q, smooth_k
from .quant_triton import fp8_block_quant, fp8_per_channel_quant, mxfp8_qk_quant, mxfp8_v_quant


@dataclass
class PreparedQKV:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    q_scale: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    qm: torch.Tensor | None = None
    k_mean: torch.Tensor | None = None
    correction: torch.Tensor | None = None
    kmeans: KMeansReorderResult | None = None


# quantizer dispatch by configuration string: (tensor, cfg) -> (codes, scale)
_QK_QUANTIZERS = {
    "fp8_block": lambda t, cfg: fp8_block_quant(t, block_s=cfg.fp8_block_size),
    "mxfp8": lambda t, cfg: mxfp8_qk_quant(t, block_d=cfg.mxfp8_block_size),
}
_V_QUANTIZERS = {
    "fp8_channel": lambda t, cfg: fp8_per_channel_quant(t),
    "fp8_block": lambda t, cfg: fp8_block_quant(t, block_s=cfg.v_fp8_block_size),
    "mxfp8": lambda t, cfg: mxfp8_v_quant(t, block_s=cfg.v_mxfp8_block_size),
}


def _checked_inputs(q, k, v):
    if not (q.shape == k.shape == v.shape):
        raise ValueError(f"q/k/v shapes must match; got {q.shape}, {k.shape}, {v.shape}")
    if q.ndim != 4:
        raise ValueError(f"q/k/v must be 4-D NHD; got {q.shape}")
    if not all(t.is_cuda for t in (q, k, v)):
        raise ValueError("q/k/v must live on CUDA")
    return q.contiguous(), k.contiguous(), v.contiguous()


def prepare_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: QuantConfig) -> PreparedQKV:
    """Preprocess (Q k-means reorder, K / Q smoothing, Hadamard) and quantise; codes and scales come back in the
    reference's shapes (pipeline.py:42-110)."""
    if cfg.smoothing not in ("off", "k_only", "full"):
        raise ValueError(f"unsupported smoothing mode: {cfg.smoothing!r}")
    if cfg.qk_quant not in _QK_QUANTIZERS:
        raise ValueError(f"unsupported qk_quant: {cfg.qk_quant!r}")
    if cfg.v_quant not in _V_QUANTIZERS:
        raise ValueError(f"unsupported v_quant: {cfg.v_quant!r}")
    qw, kw, vw = _checked_inputs(q, k, v)
    kmeans = qm = k_mean = correction = None

    if cfg.q_kmeans_k is not None:
        kmeans = q_kmeans_reorder(qw, n_clusters=cfg.q_kmeans_k, max_iters=cfg.q_kmeans_iters, seed=cfg.q_kmeans_seed)
        qw = kmeans.q_reordered
    if cfg.smoothing != "off":
        kw, k_mean = smooth_k(kw)
    if cfg.smoothing == "full":
        qw, qm = group_mean_q(qw, block_q=cfg.q_smooth_block_size)
        # the reference's einsum("bqhd,bshd->bqhs") as one FP32 product on the device
        n_keys = kw.shape[1]
        corr, _ = qm_corr(qm, kw, sm_scale=1.0, s_pad=(n_keys + 63) // 64 * 64)
        correction = corr[..., :n_keys].permute(0, 2, 1, 3).contiguous().to(cfg.correction_dtype)
    if cfg.qk_hadamard:
        qw, kw = apply_qk_hadamard(qw, kw, random_sign=cfg.qk_hadamard_random_sign, seed=cfg.qk_hadamard_seed)

    (q_codes, q_scale), (k_codes, k_scale) = (_QK_QUANTIZERS[cfg.qk_quant](t, cfg) for t in (qw, kw))
    v_codes, v_scale = _V_QUANTIZERS[cfg.v_quant](vw, cfg)
    return PreparedQKV(q=q_codes, k=k_codes, v=v_codes, q_scale=q_scale, k_scale=k_scale, v_scale=v_scale,
                       qm=qm, k_mean=k_mean, correction=correction, kmeans=kmeans)
