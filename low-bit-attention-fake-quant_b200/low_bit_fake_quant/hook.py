"""Sequence-length adapter for callers whose S does not divide the configured block sizes.

The reference's Wan2.1 attention hook (bench/wan_attention_hook.py:248-294) pads S up to the least common multiple of
the block sizes the path needs before calling ``fake_quant_attention`` and strips the padded rows afterwards: Q rows
are padded with zeros (their outputs are dropped), K / V rows replicate the last real token, so that the attention
weight falling on a padded key flows to the value of the last real token (a perturbation bounded by pad / S).
This module provides that policy for the drop-in package, and the cross-attention entry the hook has no
fake-quant form of; both are extensions, kept out of ``__all__``.
"""
from __future__ import annotations

import math
from functools import reduce
from typing import Optional

import torch

from .attention import fake_quant_attention
from .config import QuantConfig


def required_multiple(cfg: QuantConfig) -> int:
    """Least common multiple of the block sizes S has to divide for ``cfg``."""
    sizes = [cfg.fp8_block_size, cfg.v_fp8_block_size, cfg.p_requant_block_m, cfg.p_requant_block_n]
    if cfg.smoothing == "full":
        sizes.append(cfg.q_smooth_block_size)
    if cfg.v_smooth_mode == "per_block":
        sizes.append(cfg.v_smooth_block_size)
    return reduce(lambda a, b: a * b // math.gcd(a, b), sizes, 1)


def pad_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: QuantConfig):
    """``(q_padded, k_padded, v_padded, pad)``: zero Q rows, replicated last K / V row."""
    pad = -q.shape[1] % required_multiple(cfg)
    if pad == 0:
        return q, k, v, 0
    b, _, h, d = q.shape
    q_p = torch.cat((q, q.new_zeros(b, pad, h, d)), dim=1)
    k_p = torch.cat((k, k[:, -1:].expand(-1, pad, -1, -1)), dim=1)
    v_p = torch.cat((v, v[:, -1:].expand(-1, pad, -1, -1)), dim=1)
    return q_p, k_p, v_p, pad


def fake_quant_attention_padded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: Optional[QuantConfig] = None, *,
                                sm_scale: Optional[float] = None) -> torch.Tensor:
    """``fake_quant_attention`` for any S: pad by the hook's policy, run, return the first S rows."""
    if cfg is None:
        cfg = QuantConfig()
    s = q.shape[1]
    q_p, k_p, v_p, pad = pad_qkv(q, k, v, cfg)
    out = fake_quant_attention(q_p, k_p, v_p, cfg, sm_scale=sm_scale)
    return out if pad == 0 else out[:, :s].contiguous()


def fake_quant_cross_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: Optional[QuantConfig] = None, *,
                               sm_scale: Optional[float] = None) -> torch.Tensor:
    """Fake-quant attention of ``q`` (B, Sq, H, D) over ``k`` / ``v`` (B, Sk, H, D) with Sk != Sq allowed.

    An extension with no counterpart in the reference, whose entry takes equal shapes only and whose hook sends
    cross-attention to plain SDPA (bench/wan_attention_hook.py:227, 319-327). The same preprocessing order,
    quantizers and streaming kernel are used; every block size must divide the length of the tensor it applies to
    (Q-side: ``fp8_block_size``, ``p_requant_block_m``, ``q_smooth_block_size``; K / V-side: ``fp8_block_size``,
    the V block sizes, ``p_requant_block_n``, ``v_smooth_block_size``). Requires ``cfg.p_requant``.
    """
    if cfg is None:
        cfg = QuantConfig()
    return fake_quant_attention(q, k, v, cfg, sm_scale=sm_scale, _cross=True)
