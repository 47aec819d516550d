"""Fused preparation of Q, K and V for the streaming kernel (CUDA, sm_100a).

The reference prepares each tensor through a chain of full-tensor steps (src/low_bit_fake_quant/attention.py:166-239
and :505-591): k-means gather, smoothing, Hadamard rotation, quantizer, NHD -> BHSD copy. ``prep_fused`` does all of
them for one tensor in a single pass (``lbfq_prep_fused``, csrc/prep_fused.cu) and returns exactly what the separate
functions of this package return for the same steps -- codes, scales, means -- bit for bit.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib as L
from .hadamard import _cached_cpu_signs, _next_power_of_two

_KINDS = {"fp8_block": L.PREP_FP8_BLOCK, "fp8_channel": L.PREP_FP8_CHANNEL, "mxfp8_v": L.PREP_MXFP8_V, "mxfp8_qk": L.PREP_MXFP8_QK}


def group_rows(kind: str, *, smooth_block: int, scale_block: int, seq: int, dim: int, dtype: torch.dtype) -> int:
    """Rows one CTA of the fused kernel takes for these block sizes; 0 when the fused kernel does not serve them."""
    return int(L.lib().lbfq_prep_group_rows(_KINDS[kind], int(smooth_block), int(scale_block), int(seq), int(dim), L.dtype_code(dtype)))


def hadamard_signs(heads: int, dim: int, seed: int, device, *, head_offset: int = 0, total_heads: Optional[int] = None):
    """The (heads, D) +-1 table of apply_qk_hadamard for this call's heads, on the device."""
    table = _cached_cpu_signs(total_heads if total_heads is not None else heads, dim, seed)
    return table[head_offset:head_offset + heads].contiguous().to(device)


def prep_fused(x: torch.Tensor, *, kind: str, scale_block: int = 0, order: Optional[torch.Tensor] = None,
               chan_mean: Optional[torch.Tensor] = None, smooth_block: int = 0, hadamard: bool = False,
               signs: Optional[torch.Tensor] = None, layout: int = L.LAYOUT_NHD, s_pad: int = 0,
               want_scale_e8: bool = False, want_prepared: bool = False):
    """Gather (``order``), smooth (``chan_mean`` and / or ``smooth_block``), rotate (``hadamard``) and quantise
    (``kind``) the NHD tensor ``x`` in one pass.

    Returns ``(codes, scale, block_mean, scale_e8, prepared)``: ``block_mean`` (B, S/smooth_block, H, D) fp32 when
    ``smooth_block`` > 0; ``scale_e8`` the UE8M0 scale tiles (mxfp8_qk with ``want_scale_e8``); ``prepared`` the
    re-ordered, smoothed tensor in ``x``'s dtype as it is before the rotation, when ``want_prepared`` (the caller needs
    K_smooth for the score bias) -- each ``None`` otherwise."""
    if x.ndim != 4 or not x.is_cuda:
        raise ValueError(f"x must be 4-D NHD on CUDA; got {tuple(x.shape)} on {x.device}")
    b, s, h, d = x.shape
    x = x.contiguous()
    dev = x.device
    if layout == L.LAYOUT_NHD:
        shape = (b, s, h, d)
    elif layout == L.LAYOUT_BHSD:
        shape = (b, h, s_pad, d)
    else:
        shape = (b, h, d, s_pad)
    codes = torch.empty(shape, dtype=torch.float8_e4m3fn, device=dev)
    if kind == "fp8_block":
        scale = torch.empty((b, s // scale_block, h), dtype=torch.float32, device=dev)
    elif kind == "fp8_channel":
        scale = torch.empty((b, h, d), dtype=torch.float32, device=dev)
    elif kind == "mxfp8_v":
        scale = torch.empty((b, s // scale_block, h, d), dtype=torch.float32, device=dev)
    else:
        scale = torch.empty((b, s, h, d // scale_block), dtype=torch.float32, device=dev)
    block_mean = torch.empty((b, s // smooth_block, h, d), dtype=torch.float32, device=dev) if smooth_block > 0 else None
    scale_e8 = torch.empty((b * h * s_pad * 4,), dtype=torch.uint8, device=dev) if want_scale_e8 else None
    prepared = torch.empty_like(x) if want_prepared else None
    order = order.contiguous() if order is not None else None
    chan_mean = chan_mean.contiguous() if chan_mean is not None else None
    signs = signs.contiguous() if signs is not None else None
    a = L.PrepArgs()
    a.x, a.dtype = x.data_ptr(), L.dtype_code(x.dtype)
    a.B, a.S, a.H, a.D = b, s, h, d
    a.order, a.chan_mean = L.ptr(order), L.ptr(chan_mean)
    a.smooth_block, a.block_mean = int(smooth_block), L.ptr(block_mean)
    a.hadamard, a.signs = (1 if hadamard else 0), L.ptr(signs)
    a.had_scale = 1.0 / math.sqrt(float(_next_power_of_two(d)))
    a.kind, a.scale_block = _KINDS[kind], int(scale_block)
    a.codes, a.layout, a.s_pad = codes.data_ptr(), int(layout), int(s_pad)
    a.scale, a.scale_e8, a.smooth_out = scale.data_ptr(), L.ptr(scale_e8), L.ptr(prepared)
    import ctypes as C
    with torch.cuda.device(dev):
        L.check(L.lib().lbfq_prep_fused(C.byref(a), L.stream_ptr(dev)))
    return codes, scale, block_mean, scale_e8, prepared
