"""K / Q / V smoothing (CUDA, sm_100a).

Same functions and return values as src/low_bit_fake_quant/preprocess.py
(``smooth_k`` :38-57, ``smooth_v_per_block`` :135-166, ``group_mean_q``
:169-193): the centred tensor keeps the input dtype, the mean is FP32.
"""

from __future__ import annotations

from typing import Tuple

import torch

from . import _lib as L


def smooth_k(k: torch.Tensor, block_s: int = 256) -> Tuple[torch.Tensor, torch.Tensor]:
    """K minus its mean over S. Returns ``(k_smoothed, k_mean (B,H,D) fp32)``."""
    if k.ndim != 4 or not k.is_cuda:
        raise ValueError(f"k must be 4-D NHD on CUDA; got {tuple(k.shape)} on {k.device}")
    b, s, h, d = k.shape
    k = k.contiguous()
    out = torch.empty_like(k)
    mean = torch.empty((b, h, d), dtype=torch.float32, device=k.device)
    with torch.cuda.device(k.device):
        n = L.lib().lbfq_smooth_k_scratch_floats(b, s, h, d)
        partial = torch.empty((n,), dtype=torch.float32, device=k.device)
        L.check(L.lib().lbfq_smooth_k(k.data_ptr(), L.dtype_code(k.dtype), b, s, h, d, out.data_ptr(),
                                      mean.data_ptr(), partial.data_ptr(), L.stream_ptr(k.device)))
    return out, mean


def k_channel_mean(k: torch.Tensor) -> torch.Tensor:
    """The mean ``smooth_k`` subtracts, (B, H, D) fp32, without the smoothed tensor (internal: the K quantizer can
    centre on the fly)."""
    if k.ndim != 4 or not k.is_cuda:
        raise ValueError(f"k must be 4-D NHD on CUDA; got {tuple(k.shape)} on {k.device}")
    b, s, h, d = k.shape
    k = k.contiguous()
    mean = torch.empty((b, h, d), dtype=torch.float32, device=k.device)
    with torch.cuda.device(k.device):
        n = L.lib().lbfq_smooth_k_scratch_floats(b, s, h, d)
        partial = torch.empty((n,), dtype=torch.float32, device=k.device)
        L.check(L.lib().lbfq_smooth_k(k.data_ptr(), L.dtype_code(k.dtype), b, s, h, d, None,
                                      mean.data_ptr(), partial.data_ptr(), L.stream_ptr(k.device)))
    return mean


def _block_mean_sub(x: torch.Tensor, block: int, name: str) -> Tuple[torch.Tensor, torch.Tensor]:
    if x.ndim != 4 or not x.is_cuda:
        raise ValueError(f"{name} must be 4-D NHD on CUDA; got {tuple(x.shape)} on {x.device}")
    b, s, h, d = x.shape
    if s % block != 0:
        raise ValueError(f"S={s} must be divisible by block_s={block}")
    if d not in (64, 128):
        raise ValueError(f"D must be 64 or 128; got {d}")
    x = x.contiguous()
    out = torch.empty_like(x)
    mean = torch.empty((b, s // block, h, d), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        L.check(L.lib().lbfq_block_mean_sub(x.data_ptr(), L.dtype_code(x.dtype), b, s, h, d, block,
                                            out.data_ptr(), mean.data_ptr(), L.stream_ptr(x.device)))
    return out, mean


def smooth_v_per_block(v: torch.Tensor, block_s: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-S-block V mean smoothing: ``(v_centered, v_alpha (B, S/block_s, H, D) fp32)``."""
    return _block_mean_sub(v, block_s, "v")


def group_mean_q(q: torch.Tensor, block_q: int = 256) -> Tuple[torch.Tensor, torch.Tensor]:
    """Q centering by groups along S: ``(q_centered, qm (B, S/block_q, H, D) fp32)``."""
    if q.ndim == 4 and q.is_cuda and q.shape[1] % block_q != 0:
        raise ValueError(f"S={q.shape[1]} must be divisible by block_q={block_q}")
    return _block_mean_sub(q, block_q, "q")
