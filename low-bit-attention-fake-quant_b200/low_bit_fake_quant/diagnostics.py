"""Row-max update / rescale counters of the streaming attention kernel.

The reference counts these events with a diagnostic kernel of its own
(bench/count_rowmax_updates_triton.py:27-171) to show that the estimated row max (``rowmax_mode="qm_k"``) removes
most accumulator rescales. Here the production kernel counts them itself, as an opt-in epilogue of the general
kernel (``lbfq_attn_args.rowmax_counters``): what is counted is what the configured path really does, with its
own thresholds (up 16 / down 32 in log2 units for the estimated row max, any rise of the max for the online one).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .attention import _fake_quant_attention_p_requant, _preprocess
from .config import QuantConfig

COUNTER_NAMES = ("updates", "rescales", "upward_updates", "downward_updates", "rows_with_update", "max_updates_per_row")


def count_rowmax_updates(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: Optional[QuantConfig] = None, *,
                         sm_scale: Optional[float] = None) -> dict:
    """Run path B of ``fake_quant_attention`` once with the counters on; returns the reference script's report keys
    (count_rowmax_updates_triton.py:281-292) for this configuration."""
    if cfg is None:
        cfg = QuantConfig()
    if not cfg.p_requant:
        raise ValueError("row-max counters belong to the streaming kernel: requires cfg.p_requant=True")
    if q.ndim != 4 or not q.is_cuda:
        raise ValueError("q/k/v must be 4-D NHD on CUDA")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    q_work, k_work, v_work, qm, v_alpha, q_km, _ = _preprocess(q.contiguous(), k.contiguous(), v.contiguous(), cfg)
    counters = torch.zeros(6, dtype=torch.int64, device=q.device)
    _fake_quant_attention_p_requant(q_work, k_work, v_work, qm, v_alpha, q_km, cfg, sm_scale, q.dtype,
                                    rowmax_counters=counters)
    vals = [int(x) for x in counters.cpu().tolist()]
    b, s, h, _ = q.shape
    rows = b * h * s
    row_tiles = rows * ((s + cfg.p_requant_block_n - 1) // cfg.p_requant_block_n)
    out = dict(zip(COUNTER_NAMES, vals))
    out.update(updates_per_row_avg=vals[0] / rows, rescales_per_row_avg=vals[1] / rows,
               update_rate_per_row_tile=vals[0] / row_tiles, rescale_rate_per_row_tile=vals[1] / row_tiles)
    return out
