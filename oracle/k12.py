"""CPU restatement of the reference streaming attention kernel ("K12").

TEST INFRASTRUCTURE ONLY (see ``oracle/quant_ops.py``).

Follows ``_fake_quant_attn_fwd_kernel``
(src/low_bit_fake_quant/attention_triton.py:48-407) block for block: the same
per-(row, 64-key block) running max, rescale factor, P quantisation, V block
scale, V-alpha correction accumulator, estimated-row-max thresholds and BLASST
skip / fill rules, written as torch ops over all rows of a (B, H) slab at once
with a Python loop over key blocks.

Two operand conventions are supported, selected by what the caller passes:

* ``faithful`` (``row_scale is None``): Q/K are the reference's de-quantised
  BF16 operands, the recovered P is rounded to BF16 before the PV product
  (attention_triton.py:331,347,360) -- this is the reference's own arithmetic
  and is pinned by the torch mirrors in the reference's tests
  (tests/test_triton_attn.py:24-151, reproduced through ``tests/golden``).
* ``true FP8`` (``row_scale`` / ``col_scale`` given): Q/K are raw e4m3 codes,
  the logits are ``(codes @ codes^T) * ((sq * sk) * sm_scale)`` and the
  recovered P stays FP32. This is what a real FP8 tensor-core kernel computes;
  the gap to the faithful convention is the BF16 rounding of the de-quantised
  operands and is measured, not hidden.
"""

from __future__ import annotations

import math
import re
from typing import Optional, Tuple

import torch

from .quant_ops import FP8_MAX, INV_FP8_MAX, divide, pow2_scale, to_e4m3

LOG2E = 1.4426950408889634

FILL_ZERO, FILL_MAX, FILL_MEAN, FILL_LOGN, FILL_SAMPLE8, FILL_THR, FILL_UTA = range(7)


def parse_blasst_fill(mode: Optional[str], *, alpha: float, uta_bins: int) -> Tuple[int, float, int]:
    """Fill string -> (kind, alpha, bins). attention_triton.py:674-714."""
    if mode is None or mode == "zero":
        return FILL_ZERO, float(alpha), 1
    for name, kind in (("max", FILL_MAX), ("mean", FILL_MEAN), ("sample8", FILL_SAMPLE8), ("thr", FILL_THR)):
        if mode == name:
            return kind, float(alpha), 1
        if mode.startswith(name + "_a"):
            return kind, float(mode[len(name) + 2:]), 1
    if mode == "logn":
        return FILL_LOGN, float(alpha), 1
    if mode == "uta":
        if uta_bins <= 0:
            raise ValueError(f"blasst_uta_bins must be > 0; got {uta_bins}")
        return FILL_UTA, float(alpha), int(uta_bins)
    m = re.fullmatch(r"uta(\d+)(?:_a([0-9]+(?:\.[0-9]+)?))?", mode)
    if m:
        bins = int(m.group(1))
        if bins <= 0:
            raise ValueError(f"UTA bin count must be > 0; got {bins}")
        return FILL_UTA, float(m.group(2)) if m.group(2) is not None else float(alpha), bins
    raise ValueError(f"unknown blasst_fill_mode: {mode!r}")


def _f32(x: float) -> torch.Tensor:
    return torch.tensor(x, dtype=torch.float32)


def k12_attention(
    q_op: torch.Tensor,            # (B,H,M,D) fp32: dequantised Q (faithful) or raw codes (true FP8)
    k_op: torch.Tensor,            # (B,H,N,D)
    v_op: torch.Tensor,            # (B,H,N,D) raw V codes as fp32 (channel / block) or dequantised (mx)
    v_scale_bhd: torch.Tensor,     # (B,H,D) fp32, ones when unused
    *,
    sm_scale: float,
    p_max_offset: float,
    block_m: int = 64,
    block_n: int = 64,
    row_scale: Optional[torch.Tensor] = None,      # (B,H,M) per-row Q scale (true FP8)
    col_scale: Optional[torch.Tensor] = None,      # (B,H,N) per-key K scale (true FP8)
    v_alpha: Optional[torch.Tensor] = None,        # (B, N/v_smooth_block, H, D)
    v_smooth_block: int = 0,
    k_smooth: Optional[torch.Tensor] = None,       # (B,H,N,D) un-quantised smoothed K
    qm: Optional[torch.Tensor] = None,             # (B, M/q_smooth_block, H, D)
    q_smooth_block: int = 0,
    v_block_scale: Optional[torch.Tensor] = None,  # (B, N/v_block_size, H)
    v_block_size: int = 0,
    p_quant_mode: str = "elementwise",
    rowmax_est: Optional[torch.Tensor] = None,     # (B,H,M)
    rowmax_init: Optional[torch.Tensor] = None,    # (B,H,M)
    blasst_lambda: Optional[float] = None,
    blasst_fill_mode: Optional[str] = "zero",
    blasst_fill_alpha: float = 1.0,
    blasst_uta_bins: int = 16,
    blasst_tile_rows: int = 0,
    row_index: Optional[torch.Tensor] = None,
    p_probe: Optional[dict] = None,
    p_flip=None,
    faithful: Optional[bool] = None,
    p_bf16: Optional[bool] = None,
    return_stats: bool = False,
    rowmax_counters: Optional[dict] = None,
):
    """Returns FP32 output (B,H,M,D) before the final cast (and stats).

    ``rowmax_counters``: a dict that receives the row-max update counts of this run, the events the reference's
    diagnostic kernel counts (bench/count_rowmax_updates_triton.py:118-171): an update moves a row's reference max,
    a rescale is an update of a row that already holds mass.

    ``blasst_tile_rows`` > 0 replaces the kernel's row-by-row skip decision by the tile-level one of the reference's
    simulator (blasst_skip.py:573-585): a key block is dropped only when every row of a tile of that many query rows
    finds it under the threshold, and then for all of them (zero fill).

    Aids for checking a claim of the parity tests -- that a row outside the tolerance differs from this restatement
    by ONE e4m3 code step of one P value that sits on a rounding boundary: ``row_index`` (1-D int64) computes only those
    query rows (the result then has ``len(row_index)`` rows, in that order; no stats); ``p_probe`` (a dict) receives
    ``quotient`` -- what went into the e4m3 rounding, ``p`` or ``p / s_P``, (B,H,rows,N) --, ``codes``, the rounded
    values, ``p_used``, the values that entered P.V, and ``row_max``, the reference max of each key's block; ``p_flip = (row, key, step)``, or a list of such triples, moves the code of P[row, key] (row counted within the
    computed rows) by ``step`` = +1 / -1 e4m3 code steps before it is used; ``(row, key, step, "bf16")`` moves the
    BF16-rounded value ``bf16(code x s_P)`` of the scaled P modes by one BF16 ulp instead (the reference's second
    rounding, attention_triton.py:353-360)."""
    B, H, M, D = q_op.shape
    N = k_op.shape[2]
    if faithful is None:
        faithful = row_scale is None
    if p_bf16 is None:            # the reference rounds the re-scaled P to BF16 before P.V (attention_triton.py:331-360)
        p_bf16 = faithful
    pk = {"elementwise": 0, "mx": 1, "dynamic": 2}[p_quant_mode]
    use_blasst = blasst_lambda is not None
    if use_blasst:
        if not (0.0 < float(blasst_lambda) < 1.0):
            raise ValueError(f"blasst_lambda must be in (0, 1); got {blasst_lambda}")
        log_lambda = _f32(math.log(float(blasst_lambda)))
        fill_kind, fill_alpha, uta_bins = parse_blasst_fill(
            blasst_fill_mode, alpha=blasst_fill_alpha, uta_bins=blasst_uta_bins)
        if fill_kind == FILL_UTA and block_n % uta_bins != 0:
            raise ValueError(f"blasst UTA bins ({uta_bins}) must divide block_n ({block_n})")
    else:
        fill_kind, fill_alpha, uta_bins = FILL_ZERO, 1.0, 1
    if rowmax_est is not None and rowmax_init is not None:
        raise ValueError("rowmax_init_bhs and rowmax_est_bhs are mutually exclusive")

    if row_index is not None:
        if return_stats or blasst_tile_rows:
            raise ValueError("row_index computes single rows: no stats tensor, no tile-level predicate")
        row_index = row_index.to(torch.int64)
        q_op = q_op[:, :, row_index]
        row_scale = row_scale[:, :, row_index] if row_scale is not None else None
        rowmax_est = rowmax_est[:, :, row_index] if rowmax_est is not None else None
        rowmax_init = rowmax_init[:, :, row_index] if rowmax_init is not None else None
        M = int(row_index.numel())
    if p_probe is not None:
        p_probe["quotient"] = torch.zeros((B, H, M, N))
        p_probe["codes"] = torch.zeros((B, H, M, N))
        p_probe["p_scaled"] = torch.zeros((B, H, M, N))        # codes x s_P, before the BF16 rounding of the scaled modes
        p_probe["p_used"] = torch.zeros((B, H, M, N))          # the P values that entered P.V
        p_probe["row_max"] = torch.zeros((B, H, M, N))         # the reference max the key's block was taken against
    q_op = q_op.float()
    k_op = k_op.float()
    v_op = v_op.float()
    log2e = _f32(LOG2E)
    off = _f32(float(p_max_offset))
    sm = _f32(float(sm_scale))

    rows = torch.arange(M) if row_index is None else row_index
    if qm is not None:
        # attention_triton.py:121-124: one qm vector per program (M block)
        grp = ((rows // block_m) * block_m) // q_smooth_block
        qm_rows = qm.float().permute(0, 2, 1, 3)[:, :, grp, :]            # (B,H,M,D)

    if rowmax_est is not None:
        m_i = rowmax_est.float().clone()
    elif rowmax_init is not None:
        m_i = rowmax_init.float().clone()
    else:
        m_i = torch.full((B, H, M), -float("inf"))
    est = rowmax_est.float() if rowmax_est is not None else None
    l_i = torch.zeros((B, H, M))
    acc = torch.zeros((B, H, M, D))
    c_acc = torch.zeros((B, H, M, D))
    max_seen = torch.full((B, H, M), -float("inf"))
    skipped_cnt = torch.zeros((B, H, M))
    total_cnt = torch.zeros((B, H, M))
    upd_cnt = torch.zeros((B, H, M), dtype=torch.int64)
    n_resc = n_down = 0

    for n0 in range(0, N, block_n):
        n1 = min(n0 + block_n, N)
        nv = n1 - n0
        kb = k_op[:, :, n0:n1]
        s = torch.matmul(q_op, kb.transpose(-2, -1))                       # fp32 accumulate
        if row_scale is not None:
            f = (row_scale.float()[..., :, None] * col_scale.float()[:, :, None, n0:n1]) * sm
            s = s * f
        else:
            s = s * sm
        if qm is not None:
            ks = k_smooth[:, :, n0:n1].float()
            corr = torch.matmul(qm_rows, ks.transpose(-2, -1)) * sm        # :156-160
            s = s + corr

        block_max = s.amax(dim=-1)
        skip_row = torch.zeros((B, H, M), dtype=torch.bool)
        if use_blasst:                                                     # :165-175
            m_ij = torch.maximum(m_i, block_max)
            skip_row = (block_max - m_ij) < log_lambda
            if blasst_tile_rows:
                tr = int(blasst_tile_rows)
                padded = torch.nn.functional.pad(skip_row, (0, (-M) % tr), value=True)
                whole = padded.reshape(B, H, -1, tr).all(dim=-1, keepdim=True)
                skip_row = whole.expand(-1, -1, -1, tr).reshape(B, H, -1)[..., :M]
            alpha = torch.exp2((m_i - m_ij) * log2e)
            alpha = torch.where(skip_row, torch.ones_like(alpha), alpha)
            m_ij = torch.where(skip_row, m_i, m_ij)
            skipped_cnt += skip_row.float()
            total_cnt += 1.0
        elif est is not None:
            if pk == 2:                                                    # :177-211
                max_seen_ij = torch.maximum(max_seen, block_max)
                up = _f32(16.0) / log2e
                down = _f32(32.0) / log2e
                under = (block_max - m_i) > up
                over = (m_i - max_seen_ij) > down
                adjust = under | over
                down_bounded = torch.maximum(max_seen_ij + down, m_i - 80.0)
                down_m = torch.where(l_i == 0.0, max_seen_ij, down_bounded)
                adjusted = torch.where(under, block_max, down_m)
                m_ij = torch.where(adjust, adjusted, m_i)
                a_upd = torch.exp2((m_i - m_ij) * log2e)
                a_upd = torch.where(l_i == 0.0, torch.zeros_like(a_upd), a_upd)
                alpha = torch.where(adjust, a_upd, torch.ones_like(a_upd))
                max_seen = max_seen_ij
            else:                                                          # :212-214
                m_ij = est
                alpha = torch.ones((B, H, M))
        else:                                                              # :215-217
            m_ij = torch.maximum(m_i, block_max)
            alpha = torch.exp2((m_i - m_ij) * log2e)

        if rowmax_counters is not None:
            moved = m_ij != m_i
            if est is not None and pk == 2 and not use_blasst:
                n_down += int((moved & ~((block_max - m_i) > _f32(16.0) / log2e)).sum())
            else:
                moved = m_ij > m_i
            upd_cnt += moved.long()
            n_resc += int((moved & (l_i != 0.0)).sum())

        if pk == 0:
            z = (s - m_ij[..., None]) * log2e + off
        else:
            z = (s - m_ij[..., None]) * log2e
        p = torch.exp2(z)

        if use_blasst:
            if fill_kind == FILL_ZERO:
                p = torch.where(skip_row[..., None], torch.zeros_like(p), p)
            else:
                p_exact = torch.where(skip_row[..., None], torch.zeros_like(p), p)
                safe_n = _f32(float(max(nv, 1)))
                fill_off = off if pk == 0 else _f32(0.0)
                mean = s.sum(dim=-1) / safe_n
                max_bound = safe_n * torch.exp2((block_max - m_ij) * log2e + fill_off)
                a = _f32(fill_alpha)
                if fill_kind == FILL_MAX:
                    fill_p = (max_bound * a / safe_n)[..., None].expand_as(s)
                elif fill_kind == FILL_MEAN:
                    mass = a * safe_n * torch.exp2((mean - m_ij) * log2e + fill_off)
                    fill_p = (torch.minimum(mass, max_bound) / safe_n)[..., None].expand_as(s)
                elif fill_kind == FILL_LOGN:
                    cen = s - mean[..., None]
                    var = (cen * cen).sum(dim=-1) / safe_n
                    mass = safe_n * torch.exp2((mean + 0.5 * var - m_ij) * log2e + fill_off)
                    fill_p = (torch.minimum(mass, max_bound) / safe_n)[..., None].expand_as(s)
                elif fill_kind == FILL_SAMPLE8:
                    stride = block_n // 8 if block_n >= 8 else 1
                    rel = torch.arange(nv)
                    smask = (rel % stride) == 0
                    cnt = _f32(float(max(int(smask.sum()), 1)))
                    sp = torch.exp2((s - m_ij[..., None]) * log2e + fill_off)
                    sp = torch.where(smask, sp, torch.zeros_like(sp))
                    mass = a * safe_n * sp.sum(dim=-1) / cnt
                    fill_p = (torch.minimum(mass, max_bound) / safe_n)[..., None].expand_as(s)
                elif fill_kind == FILL_THR:
                    off_scale = torch.exp2(off) if pk == 0 else _f32(1.0)
                    mass = a * safe_n * _f32(float(blasst_lambda)) * off_scale
                    fill_p = (mass / safe_n).expand_as(s)
                else:                                                      # UTA :297-323
                    bin_size = block_n // uta_bins
                    fill_p = torch.zeros_like(s)
                    for bi in range(uta_bins):
                        c0, c1 = bi * bin_size, min((bi + 1) * bin_size, nv)
                        if c1 <= c0:
                            continue
                        cnt = _f32(float(c1 - c0))
                        sb = s[..., c0:c1]
                        b_mean = sb.sum(dim=-1) / cnt
                        b_max = sb.amax(dim=-1)
                        b_bound = cnt * torch.exp2((b_max - m_ij) * log2e + fill_off)
                        b_mass = a * cnt * torch.exp2((b_mean - m_ij) * log2e + fill_off)
                        b_p = torch.minimum(b_mass, b_bound) / cnt
                        fill_p[..., c0:c1] = b_p[..., None]
                p = p_exact + torch.where(skip_row[..., None], fill_p, torch.zeros_like(s))

        l_i = l_i * alpha + p.sum(dim=-1)                                  # :326 (pre-quantisation p)

        flips = [p_flip] if isinstance(p_flip, tuple) else (p_flip or [])

        def rounded(quotient):
            codes = to_e4m3(quotient).float()
            for r_f, key_f, step_f, *kind_f in flips:
                if not kind_f and n0 <= key_f < n1:
                    c_f = key_f - n0
                    bits = codes[..., r_f, c_f].to(torch.float8_e4m3fn).view(torch.uint8).to(torch.int16) + int(step_f)
                    codes[..., r_f, c_f] = bits.clamp(0, 0x7E).to(torch.uint8).view(torch.float8_e4m3fn).float()
            if p_probe is not None:
                p_probe["quotient"][..., n0:n1] = quotient
                p_probe["codes"][..., n0:n1] = codes
            return codes

        if pk == 0:                                                        # :331
            p_rec = rounded(p)
        elif pk == 1:                                                      # :338-347
            amax = p.abs().amax(dim=-1).clamp_min(1e-4)
            s_p = pow2_scale(amax)
            p_rec = rounded(p / s_p[..., None]) * s_p[..., None]
        else:                                                              # :353-360
            amax = p.abs().amax(dim=-1).clamp_min(1e-12)
            s_p = amax * INV_FP8_MAX              # the GPU's `amax / 448` (see oracle/quant_ops.py)
            p_rec = rounded(divide(p, s_p[..., None])) * s_p[..., None]
        if p_probe is not None:
            p_probe["p_scaled"][..., n0:n1] = p_rec
        if p_bf16:
            p_rec = p_rec.to(torch.bfloat16).float()
            for r_f, key_f, step_f, *kind_f in flips:                      # ("bf16",): one BF16 ulp of the rounded value
                if kind_f and kind_f[0] == "bf16" and n0 <= key_f < n1:
                    bits = p_rec[..., r_f, key_f - n0].to(torch.bfloat16).view(torch.int16) + int(step_f)
                    p_rec[..., r_f, key_f - n0] = bits.view(torch.bfloat16).float()
        if p_probe is not None:
            p_probe["p_used"][..., n0:n1] = p_rec
            p_probe["row_max"][..., n0:n1] = m_ij[..., None]

        pv = torch.matmul(p_rec, v_op[:, :, n0:n1])                        # :363
        if v_block_scale is not None:                                      # :365-372
            s_v = v_block_scale.float()[:, n0 // v_block_size, :]          # (B,H)
            pv = pv * s_v[..., None, None]
        acc = acc * alpha[..., None] + pv                                  # :376
        if v_alpha is not None:                                            # :378-383
            a_v = v_alpha.float()[:, n0 // v_smooth_block]                 # (B,H,D)
            c_acc = c_acc * alpha[..., None] + p_rec.sum(dim=-1)[..., None] * a_v[:, :, None, :]
        m_i = m_ij

    if rowmax_counters is not None:
        n_upd = int(upd_cnt.sum())
        rowmax_counters.update(updates=n_upd, rescales=n_resc, upward_updates=n_upd - n_down, downward_updates=n_down,
                               rows_with_update=int((upd_cnt > 0).sum()), max_updates_per_row=int(upd_cnt.max()))
    inv_l = divide(torch.ones(()), l_i[..., None])                                        # :387-399
    out_main = acc * v_scale_bhd.float()[:, :, None, :] if v_block_scale is None else acc
    out = (out_main + c_acc) * inv_l if v_alpha is not None else out_main * inv_l
    if return_stats:
        nmb = (M + block_m - 1) // block_m
        pad = nmb * block_m - M
        sk = torch.nn.functional.pad(skipped_cnt, (0, pad)).reshape(B * H, nmb, block_m).sum(-1)
        tt = torch.nn.functional.pad(total_cnt, (0, pad)).reshape(B * H, nmb, block_m).sum(-1)
        stats = torch.stack((sk, tt), dim=-1).permute(1, 0, 2).contiguous()   # (nmb, B*H, 2)
        return out, stats
    return out
