"""Sequence-length adapter for callers whose S does not divide the configured block sizes.

The reference's Wan2.1 attention hook (bench/wan_attention_hook.py:248-294) pads S up to the least common multiple of
the block sizes the path needs before calling ``fake_quant_attention`` and strips the padded rows afterwards: Q rows
are padded with zeros (their outputs are dropped), K / V rows replicate the last real token, so that the attention
weight falling on a padded key flows to the value of the last real token (a perturbation bounded by pad / S).
This module provides that policy for the drop-in package, the cross-attention entry the hook has no fake-quant form
of, the space-time block reorder of the reference's BLASST evaluation, and the hook itself: the dispatcher that
replaces Wan2.1's attention function, its call log and its environment-driven dump / compare switches. All of it sits
outside the reference's package (in its ``bench/``), so it is kept out of ``__all__`` here.
"""
from __future__ import annotations

import math
import os
import threading
from dataclasses import replace
from functools import reduce
from pathlib import Path
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .attention import fake_quant_attention, prepare_for_attention
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
                                   order: torch.Tensor, *, sm_scale: Optional[float] = None, **kwargs) -> torch.Tensor:
    """``fake_quant_attention`` on the tokens taken in ``order`` (a permutation of range(S), e.g.
    ``space_time_block_order``), result returned in the original token order. Exact attention does not depend on the
    order; the fake-quant one does through its per-block scales, and BLASST through which rows share a block.
    Further keywords go to ``fake_quant_attention``."""
    from .kmeans import apply_kv_permutation
    b, s, h, _ = q.shape
    if order.ndim != 1 or order.numel() != s:
        raise ValueError(f"order must be a permutation of the {s} tokens; got shape {tuple(order.shape)}")
    order = order.to(device=q.device, dtype=torch.int64)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(s, device=q.device, dtype=torch.int64)
    fwd = order.unsqueeze(0).expand(b * h, s).contiguous()
    out = fake_quant_attention(apply_kv_permutation(q, fwd), apply_kv_permutation(k, fwd), apply_kv_permutation(v, fwd),
                               cfg, sm_scale=sm_scale, **kwargs)
    return apply_kv_permutation(out, inverse.unsqueeze(0).expand(b * h, s).contiguous())


# --- the Wan2.1 attention hook itself (bench/wan_attention_hook.py:36-348 of the reference) ------------------------
#
# The reference patches ``wan.modules.attention.{attention, flash_attention}`` with a dispatcher that sends video
# self-attention (Lq == Lk > 1024) through ``fake_quant_attention`` -- padded by the policy above -- and everything
# else (cross-attention; self-attention while no configuration is set) through plain SDPA, keeps a log of every call
# and, driven by environment variables, dumps the Q / K / V of chosen calls and compares each result with SDPA or
# with the same configuration on the online row max. The same dispatcher, state, record keys and switches:
#   WAN_ATTENTION_DUMP_DIR / WAN_ATTENTION_DUMP_CALLS / WAN_ATTENTION_DUMP_LIMIT   (:58-90)
#   WAN_ATTENTION_COMPARE_SDPA=1                                                    (:93-131)
#   WAN_ATTENTION_COMPARE_ONLINE_ROWMAX=1                                           (:134-182)

_state_lock = threading.Lock()
_current_cfg: Optional[QuantConfig] = None
_call_log: list = []
NO_QUANT: Optional[QuantConfig] = None          # "no quantisation: plain SDPA"
# what runs a fake-quant call; tests on machines without a GPU substitute a stand-in of the same signature
_attention_fn: Callable = fake_quant_attention
_prepare_fn: Callable = prepare_for_attention


def set_quant_cfg(cfg: Optional[QuantConfig]) -> None:
    """Set the active QuantConfig (``None``: plain SDPA) and clear the call log (wan_attention_hook.py:43-48)."""
    global _current_cfg
    with _state_lock:
        _current_cfg = cfg
        _call_log.clear()


def get_call_log() -> list:
    with _state_lock:
        return list(_call_log)


def _log_call(record: dict) -> None:
    with _state_lock:
        _call_log.append(record)


def _maybe_dump_qkv(q, k, v, record: dict) -> None:
    dump_dir = os.environ.get("WAN_ATTENTION_DUMP_DIR")
    if not dump_dir:
        return
    with _state_lock:
        log_idx = len(_call_log)
        dump_idx = sum(1 for item in _call_log if item.get("dumped_qkv"))
    dump_calls = os.environ.get("WAN_ATTENTION_DUMP_CALLS")
    if dump_calls:
        if log_idx not in {int(item) for item in dump_calls.split(",") if item.strip()}:
            return
    elif dump_idx >= int(os.environ.get("WAN_ATTENTION_DUMP_LIMIT", "1")):
        return
    if dump_idx >= int(os.environ.get("WAN_ATTENTION_DUMP_LIMIT", "1000000")):
        return
    out_dir = Path(dump_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    path = out_dir / f"call_{log_idx:03d}.pt"
    torch.save({"query": q.detach().cpu(), "key": k.detach().cpu(), "value": v.detach().cpu(), "record": record}, path)
    record["dumped_qkv"] = str(path)


def _difference(out: torch.Tensor, ref: torch.Tensor) -> dict:
    a, b = out.float().flatten(), ref.float().flatten()
    diff = a - b
    a_norm, b_norm = torch.linalg.vector_norm(a), torch.linalg.vector_norm(b)
    return {"mse": float(diff.pow(2).mean().item()),
            "cosine": float((torch.dot(a, b) / torch.clamp(a_norm * b_norm, min=1e-12)).item()),
            "max_abs": float(diff.abs().max().item()), "out_norm": float(a_norm.item()), "ref_norm": float(b_norm.item()),
            "out_has_nan": bool(torch.isnan(out).any().item()), "out_has_inf": bool(torch.isinf(out).any().item())}


def _sdpa(q, k, v, *, dropout_p: float, causal: bool, scale: float) -> torch.Tensor:
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=dropout_p,
                                         is_causal=causal, scale=scale)
    return out.transpose(1, 2).contiguous()


def wan_attention(q, k, v, q_lens=None, k_lens=None, dropout_p: float = 0.0, softmax_scale: Optional[float] = None,
                  q_scale: Optional[float] = None, causal: bool = False, window_size=(-1, -1), deterministic: bool = False,
                  dtype: torch.dtype = torch.bfloat16, fa_version=None, version=None) -> torch.Tensor:
    """Replacement for ``wan.modules.attention.attention`` / ``flash_attention`` (wan_attention_hook.py:203-327).

    ``q, k, v``: (B, L, N, C), the NHD layout. Video self-attention (``Lq == Lk > 1024``) with a configuration set goes
    through the fake-quant path, padded to the block sizes and stripped again; everything else through plain SDPA."""
    b, lq, nq, c = q.shape
    lk = k.shape[1]
    cfg = _current_cfg
    is_self = lq == lk and lq > 1024
    half = (torch.float16, torch.bfloat16)
    q, k, v = (t if t.dtype in half else t.to(dtype) for t in (q, k, v))
    if q_scale is not None:
        q = q * q_scale
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(c)
    if is_self and cfg is not None:
        q_p, k_p, v_p, pad = pad_qkv(q, k, v, cfg)
        record = {"kind": "self-fq", "Lq": lq, "Lk": lk, "D": c, "H": nq, "pad": pad}
        _maybe_dump_qkv(q, k, v, record)
        compare_online = os.environ.get("WAN_ATTENTION_COMPARE_ONLINE_ROWMAX") == "1" and cfg.rowmax_mode == "qm_k"
        cache = _prepare_fn(q_p, k_p, v_p, cfg) if compare_online else None
        out = _attention_fn(q_p, k_p, v_p, cfg, sm_scale=softmax_scale, preprocess_cache=cache)[:, :lq]
        if os.environ.get("WAN_ATTENTION_COMPARE_SDPA") == "1":
            record["compare_sdpa"] = _difference(out, _sdpa(q, k, v, dropout_p=dropout_p, causal=causal, scale=softmax_scale))
        if compare_online:
            ref = _attention_fn(q_p, k_p, v_p, replace(cfg, rowmax_mode="online"), sm_scale=softmax_scale,
                                preprocess_cache=cache)[:, :lq]
            rec = _difference(out, ref)
            rec.update(ref_has_nan=bool(torch.isnan(ref).any().item()), ref_has_inf=bool(torch.isinf(ref).any().item()))
            record["compare_online_rowmax"] = rec
        _log_call(record)
        return out.to(q.dtype)
    out = _sdpa(q, k, v, dropout_p=dropout_p, causal=causal, scale=softmax_scale)
    _log_call({"kind": "self-sdpa" if is_self else "cross-sdpa", "Lq": lq, "Lk": lk, "D": c, "H": nq})
    return out.to(q.dtype)


_installed = False


def install_hook(attention_module=None, model_module=None) -> None:
    """Patch Wan2.1's attention entry points with :func:`wan_attention` (wan_attention_hook.py:336-348).

    Without arguments the modules ``wan.modules.attention`` and ``wan.modules.model`` are imported (the Wan2.1 code
    base has to be installed); a caller may hand them in instead."""
    global _installed
    if _installed and attention_module is None:
        return
    if attention_module is None:
        import wan.modules.attention as attention_module      # noqa: F811
        import wan.modules.model as model_module               # noqa: F811
    attention_module.attention = wan_attention
    attention_module.flash_attention = wan_attention
    if model_module is not None:
        model_module.flash_attention = wan_attention
    _installed = True
