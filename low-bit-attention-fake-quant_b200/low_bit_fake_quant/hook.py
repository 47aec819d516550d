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


# --- space-time block order (bench/eval_blasst_quant.py:101-134 of the reference) ---------------------------------
#
# Video tokens arrive flattened row-major over a (t, h, w) grid, so 64 consecutive tokens are a thin strip of one
# row. Grouping the tokens of each (ts, hs, ws) brick together makes every block of queries and keys spatially
# compact, which is what lets BLASST skip whole blocks for whole groups of rows. The order is a plain permutation
# applied to Q, K and V alike; the attention output is brought back to the original order afterwards.

def space_time_block_order(t: int, h: int, w: int, *, ts: int, hs: int, ws: int, tail: int = 0,
                           device: Optional[torch.device] = None) -> torch.Tensor:
    """Token order, brick by brick (bricks row-major over the grid, tokens row-major inside a brick; bricks cut by
    the grid's edge keep the tokens they have). ``tail`` tokens beyond the grid stay at the end, in place."""
    if min(t, h, w, ts, hs, ws) <= 0 or tail < 0:
        raise ValueError("grid and brick sizes must be positive")
    tt, hh, ww = torch.meshgrid(torch.arange(t, device=device), torch.arange(h, device=device),
                                torch.arange(w, device=device), indexing="ij")
    n_h, n_w = -(-h // hs), -(-w // ws)
    brick = ((tt // ts) * n_h + hh // hs) * n_w + ww // ws
    inner = ((tt % ts) * hs + hh % hs) * ws + ww % ws
    order = torch.argsort((brick * (ts * hs * ws) + inner).reshape(-1), stable=True)
    if tail > 0:
        order = torch.cat((order, torch.arange(t * h * w, t * h * w + tail, device=order.device)))
    return order.contiguous()


def fake_quant_attention_reordered(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: Optional[QuantConfig],
                                   order: torch.Tensor, *, sm_scale: Optional[float] = None) -> torch.Tensor:
    """``fake_quant_attention`` on the tokens taken in ``order`` (a permutation of range(S), e.g.
    ``space_time_block_order``), result returned in the original token order. Exact attention does not depend on the
    order; the fake-quant one does through its per-block scales, and BLASST through which rows share a block."""
    from .kmeans import apply_kv_permutation
    b, s, h, _ = q.shape
    if order.ndim != 1 or order.numel() != s:
        raise ValueError(f"order must be a permutation of the {s} tokens; got shape {tuple(order.shape)}")
    order = order.to(device=q.device, dtype=torch.int64)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(s, device=q.device, dtype=torch.int64)
    fwd = order.unsqueeze(0).expand(b * h, s).contiguous()
    out = fake_quant_attention(apply_kv_permutation(q, fwd), apply_kv_permutation(k, fwd), apply_kv_permutation(v, fwd),
                               cfg, sm_scale=sm_scale)
    return apply_kv_permutation(out, inverse.unsqueeze(0).expand(b * h, s).contiguous())
