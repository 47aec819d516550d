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


def prepare_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: QuantConfig) -> PreparedQKV:
    """Run the configured QKV preprocessing and quantization pipeline."""
    if q.shape != k.shape or q.shape != v.shape:
        raise ValueError(f"q/k/v shapes must match; got {q.shape}, {k.shape}, {v.shape}")
    if q.ndim != 4:
        raise ValueError(f"q/k/v must be 4-D NHD; got {q.shape}")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("q/k/v must live on CUDA")
    res = PreparedQKV(q=None, k=None, v=None, q_scale=None, k_scale=None, v_scale=None)  # type: ignore[arg-type]
    q_work, k_work, v_work = q.contiguous(), k.contiguous(), v.contiguous()

    if cfg.q_kmeans_k is not None:
        res.kmeans = q_kmeans_reorder(q_work, n_clusters=cfg.q_kmeans_k, max_iters=cfg.q_kmeans_iters,
                                      seed=cfg.q_kmeans_seed)
        q_work = res.kmeans.q_reordered

    if cfg.smoothing in ("k_only", "full"):
        k_work, res.k_mean = smooth_k(k_work)
        if cfg.smoothing == "full":
            q_work, res.qm = group_mean_q(q_work, block_q=cfg.q_smooth_block_size)
            # einsum("bqhd,bshd->bqhs") of the reference, as one fp32 product on the device
            s = k_work.shape[1]
            corr, _ = qm_corr(res.qm, k_work, sm_scale=1.0, s_pad=(s + 63) // 64 * 64)
            res.correction = corr[..., :s].permute(0, 2, 1, 3).contiguous().to(cfg.correction_dtype)
    elif cfg.smoothing != "off":
        raise ValueError(f"unsupported smoothing mode: {cfg.smoothing!r}")

    if cfg.qk_hadamard:
        q_work, k_work = apply_qk_hadamard(q_work, k_work, random_sign=cfg.qk_hadamard_random_sign,
                                           seed=cfg.qk_hadamard_seed)

    if cfg.qk_quant == "fp8_block":
        res.q, res.q_scale = fp8_block_quant(q_work, block_s=cfg.fp8_block_size)
        res.k, res.k_scale = fp8_block_quant(k_work, block_s=cfg.fp8_block_size)
    elif cfg.qk_quant == "mxfp8":
        res.q, res.q_scale = mxfp8_qk_quant(q_work, block_d=cfg.mxfp8_block_size)
        res.k, res.k_scale = mxfp8_qk_quant(k_work, block_d=cfg.mxfp8_block_size)
    else:
        raise ValueError(f"unsupported qk_quant: {cfg.qk_quant!r}")

    if cfg.v_quant == "fp8_channel":
        res.v, res.v_scale = fp8_per_channel_quant(v_work)
    elif cfg.v_quant == "fp8_block":
        res.v, res.v_scale = fp8_block_quant(v_work, block_s=cfg.v_fp8_block_size)
    elif cfg.v_quant == "mxfp8":
        res.v, res.v_scale = mxfp8_v_quant(v_work, block_s=cfg.v_mxfp8_block_size)
    else:
        raise ValueError(f"unsupported v_quant: {cfg.v_quant!r}")
    return res
