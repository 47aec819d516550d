"""FP8 / MXFP8 quantizers and de-quantizers (CUDA, sm_100a).

Same names, signatures, return shapes and error behaviour as the reference
module of this name (src/low_bit_fake_quant/quant_triton.py:15-416); the
Triton kernels are replaced by ``liblbfq.so`` (csrc/quant.cu). The module name
is kept so that ``from low_bit_fake_quant.quant_triton import ...`` keeps
working; nothing here uses Triton.
"""

from __future__ import annotations

from typing import Tuple

import torch

from . import _lib as L


def _check_nhd(t: torch.Tensor, *, name: str = "tensor") -> tuple[int, int, int, int]:
    if t.ndim != 4:
        raise ValueError(f"{name} must be 4-D NHD (B, S, H, D); got {tuple(t.shape)}")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on CUDA; got {t.device}")
    b, s, h, d = t.shape
    if d not in (64, 128):
        raise ValueError(f"{name}.shape[-1] must be 64 or 128; got {d}")
    return b, s, h, d


def _codes_like(t: torch.Tensor, layout: int, s_pad: int) -> torch.Tensor:
    b, s, h, d = t.shape
    if layout == L.LAYOUT_NHD:
        shape = (b, s, h, d)
    elif layout == L.LAYOUT_BHSD:
        shape = (b, h, s_pad, d)
    else:
        shape = (b, h, d, s_pad)
    return torch.empty(shape, dtype=torch.float8_e4m3fn, device=t.device)


def fp8_block_quant(t: torch.Tensor, block_s: int = 128, *, _layout: int = L.LAYOUT_NHD,
                    _s_pad: int = 0, _mean: torch.Tensor | None = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """FP32-scale FP8 e4m3fn quantization per (B, S/block_s, H).

    ``_mean`` (fp32 (B, H, D), internal): quantise ``(t - mean).to(t.dtype)`` without storing it (K smoothing fused
    into the K quantizer; the same codes and scales as the two steps)."""
    b, s, h, d = _check_nhd(t)
    if s % block_s != 0:
        raise ValueError(f"S={s} must be divisible by block_s={block_s}")
    t = t.contiguous()
    out = _codes_like(t, _layout, _s_pad)
    scale = torch.empty((b, s // block_s, h), dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        if _mean is not None:
            if tuple(_mean.shape) != (b, h, d) or _mean.dtype != torch.float32:
                raise ValueError(f"mean must be fp32 {(b, h, d)}; got {_mean.dtype} {tuple(_mean.shape)}")
            L.check(L.lib().lbfq_fp8_block_quant_centered(t.data_ptr(), L.dtype_code(t.dtype), b, s, h, d, block_s,
                                                          _mean.contiguous().data_ptr(), out.data_ptr(), _layout, _s_pad,
                                                          scale.data_ptr(), L.stream_ptr(t.device)))
        else:
            L.check(L.lib().lbfq_fp8_block_quant(t.data_ptr(), L.dtype_code(t.dtype), b, s, h, d, block_s,
                                                 out.data_ptr(), _layout, _s_pad, scale.data_ptr(),
                                                 L.stream_ptr(t.device)))
    return out, scale


def fp8_block_dequant(fp8: torch.Tensor, scale: torch.Tensor, block_s: int = 128, *,
                      dtype: torch.dtype = torch.float32) -> torch.Tensor:
    b, s, h, d = _check_nhd(fp8, name="fp8")
    if fp8.dtype != torch.float8_e4m3fn:
        raise TypeError(f"fp8 must have dtype torch.float8_e4m3fn; got {fp8.dtype}")
    if tuple(scale.shape) != (b, s // block_s, h):
        raise ValueError(f"scale must have shape {(b, s // block_s, h)}; got {tuple(scale.shape)}")
    fp8 = fp8.contiguous()
    scale = scale.contiguous().float()
    out = torch.empty((b, s, h, d), dtype=dtype, device=fp8.device)
    with torch.cuda.device(fp8.device):
        L.check(L.lib().lbfq_fp8_block_dequant(fp8.data_ptr(), scale.data_ptr(), b, s, h, d, block_s,
                                               out.data_ptr(), L.dtype_code(dtype), L.stream_ptr(fp8.device)))
    return out


def fp8_per_channel_quant(t: torch.Tensor, block_s: int = 128, *, _layout: int = L.LAYOUT_NHD,
                          _s_pad: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """FP32-scale FP8 e4m3fn quantization for V, one scale per (B, H, D)."""
    b, s, h, d = _check_nhd(t)
    t = t.contiguous()
    out = _codes_like(t, _layout, _s_pad)
    scale = torch.empty((b, h, d), dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        L.check(L.lib().lbfq_fp8_channel_quant(t.data_ptr(), L.dtype_code(t.dtype), b, s, h, d,
                                               out.data_ptr(), _layout, _s_pad, scale.data_ptr(),
                                               L.stream_ptr(t.device)))
    return out, scale


def fp8_per_channel_dequant(fp8: torch.Tensor, scale: torch.Tensor, block_s: int = 128, *,
                            dtype: torch.dtype = torch.float32) -> torch.Tensor:
    b, s, h, d = _check_nhd(fp8, name="fp8")
    if tuple(scale.shape) != (b, h, d):
        raise ValueError(f"scale must have shape {(b, h, d)}; got {tuple(scale.shape)}")
    fp8 = fp8.contiguous()
    scale = scale.contiguous().float()
    out = torch.empty((b, s, h, d), dtype=dtype, device=fp8.device)
    with torch.cuda.device(fp8.device):
        L.check(L.lib().lbfq_fp8_channel_dequant(fp8.data_ptr(), scale.data_ptr(), b, s, h, d,
                                                 out.data_ptr(), L.dtype_code(dtype), L.stream_ptr(fp8.device)))
    return out


def mxfp8_qk_quant(t: torch.Tensor, block_d: int = 32, *, _layout: int = L.LAYOUT_NHD, _s_pad: int = 0,
                   _scale_e8: torch.Tensor | None = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP8-style Q/K quantization along D, scale shape (B, S, H, D/block_d)."""
    b, s, h, d = _check_nhd(t)
    if d % block_d != 0:
        raise ValueError(f"D={d} must be divisible by block_d={block_d}")
    t = t.contiguous()
    out = _codes_like(t, _layout, _s_pad)
    scale = torch.empty((b, s, h, d // block_d), dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        L.check(L.lib().lbfq_mxfp8_qk_quant(t.data_ptr(), L.dtype_code(t.dtype), b, s, h, d, block_d,
                                            out.data_ptr(), _layout, _s_pad, scale.data_ptr(),
                                            L.ptr(_scale_e8), L.stream_ptr(t.device)))
    return out, scale


def mxfp8_qk_dequant(fp8: torch.Tensor, scale: torch.Tensor, block_d: int = 32, *,
                     dtype: torch.dtype = torch.float32) -> torch.Tensor:
    b, s, h, d = _check_nhd(fp8, name="fp8")
    d_blocks = d // block_d
    if tuple(scale.shape) != (b, s, h, d_blocks):
        raise ValueError(f"scale must have shape {(b, s, h, d_blocks)}")
    fp8 = fp8.contiguous()
    scale = scale.contiguous().float()
    out = torch.empty((b, s, h, d), dtype=dtype, device=fp8.device)
    with torch.cuda.device(fp8.device):
        L.check(L.lib().lbfq_mxfp8_qk_dequant(fp8.data_ptr(), scale.data_ptr(), b, s, h, d, block_d,
                                              out.data_ptr(), L.dtype_code(dtype), L.stream_ptr(fp8.device)))
    return out


def mxfp8_v_quant(t: torch.Tensor, block_s: int = 32, *, _layout: int = L.LAYOUT_NHD,
                  _s_pad: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP8-style V quantization along S, scale shape (B, S/block_s, H, D)."""
    b, s, h, d = _check_nhd(t)
    if s % block_s != 0:
        raise ValueError(f"S={s} must be divisible by block_s={block_s}")
    t = t.contiguous()
    out = _codes_like(t, _layout, _s_pad)
    scale = torch.empty((b, s // block_s, h, d), dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        L.check(L.lib().lbfq_mxfp8_v_quant(t.data_ptr(), L.dtype_code(t.dtype), b, s, h, d, block_s,
                                           out.data_ptr(), _layout, _s_pad, scale.data_ptr(),
                                           L.stream_ptr(t.device)))
    return out, scale


def mxfp8_v_dequant(fp8: torch.Tensor, scale: torch.Tensor, block_s: int = 32, *,
                    dtype: torch.dtype = torch.float32) -> torch.Tensor:
    b, s, h, d = _check_nhd(fp8, name="fp8")
    if tuple(scale.shape) != (b, s // block_s, h, d):
        raise ValueError(f"scale must have shape {(b, s // block_s, h, d)}")
    fp8 = fp8.contiguous()
    scale = scale.contiguous().float()
    out = torch.empty((b, s, h, d), dtype=dtype, device=fp8.device)
    with torch.cuda.device(fp8.device):
        L.check(L.lib().lbfq_mxfp8_v_dequant(fp8.data_ptr(), scale.data_ptr(), b, s, h, d, block_s,
                                             out.data_ptr(), L.dtype_code(dtype), L.stream_ptr(fp8.device)))
    return out
