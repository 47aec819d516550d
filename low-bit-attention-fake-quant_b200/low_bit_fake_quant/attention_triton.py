"""Launcher of the streaming fake-quant attention kernel (CUDA, sm_100a).

Takes the place of ``fake_quant_attention_triton`` and ``_parse_blasst_fill``
(src/low_bit_fake_quant/attention_triton.py:410-714). The module name is kept
for import compatibility; the kernel is ``csrc/attention.cu`` (tcgen05 FP8
MMAs, TMA, TMEM), reached through ``lbfq_attention_fwd``.

The reference launcher takes de-quantised BF16 operands; the kernel here
multiplies the e4m3 codes themselves, so its native entry point,
:func:`fake_quant_attention_fp8`, takes codes plus scales. Argument names,
validation rules, error messages, the P / V / row-max / BLASST modes and the
stats tensor contract are the reference's.
"""

from __future__ import annotations

import ctypes as C
import re
from typing import Optional

import torch

from . import _lib as L

_BLASST_FILL_ZERO = 0
_BLASST_FILL_MAX = 1
_BLASST_FILL_MEAN = 2
_BLASST_FILL_LOGN = 3
_BLASST_FILL_SAMPLE8 = 4
_BLASST_FILL_THR = 5
_BLASST_FILL_UTA = 6

# When set to a list, every launch appends a (start, end) pair of CUDA events recorded
# on the launching stream around the attention kernel (used by bench.py for the roofline).
KERNEL_EVENTS: Optional[list] = None

_status_for = L.status_for
raise_if_device_error = L.raise_if_device_error


def _parse_blasst_fill(mode: Optional[str], *, alpha: float, uta_bins: int) -> tuple[int, float, int]:
    """BLASST fill string -> (kind, alpha, bins); accepts ``mean`` + alpha as
    well as the probe spellings ``mean_a1.5`` / ``uta16_a1.5``."""
    if mode is None or mode == "zero":
        return _BLASST_FILL_ZERO, float(alpha), 1
    plain = {"max": _BLASST_FILL_MAX, "mean": _BLASST_FILL_MEAN, "logn": _BLASST_FILL_LOGN,
             "sample8": _BLASST_FILL_SAMPLE8, "thr": _BLASST_FILL_THR}
    if mode in plain:
        return plain[mode], float(alpha), 1
    for name in ("max", "mean", "sample8", "thr"):
        if mode.startswith(name + "_a"):
            return plain[name], float(mode[len(name) + 2:]), 1
    if mode == "uta":
        if uta_bins <= 0:
            raise ValueError(f"blasst_uta_bins must be > 0; got {uta_bins}")
        return _BLASST_FILL_UTA, float(alpha), int(uta_bins)
    m = re.fullmatch(r"uta(\d+)(?:_a([0-9]+(?:\.[0-9]+)?))?", mode)
    if m:
        bins = int(m.group(1))
        if bins <= 0:
            raise ValueError(f"UTA bin count must be > 0; got {bins}")
        return _BLASST_FILL_UTA, (float(m.group(2)) if m.group(2) is not None else float(alpha)), bins
    raise ValueError(f"unknown blasst_fill_mode: {mode!r}")


def fake_quant_attention_fp8(
    q_codes: torch.Tensor,          # (B, H, m_pad, D) e4m3
    k_codes: torch.Tensor,          # (B, H, n_pad, D) e4m3
    v_codes_t: torch.Tensor,        # (B, H, D, n_pad) e4m3 (keys contiguous)
    *,
    seq_q: int,
    seq_k: int,
    q_scale: Optional[torch.Tensor],   # (B, M/qk_block, H) fp32
    k_scale: Optional[torch.Tensor],   # (B, N/qk_block, H) fp32
    qk_block: int,
    operands_bf16: bool = False,    # q/k/v are BF16 (de-quantised Q/K, BF16 V^T): the reference's own operand convention
    qk_bf16_v_codes: bool = False,  # q/k are BF16 as above, v_codes_t stays e4m3 codes with its v_kind / v_scale (general kernel)
    q_scale_e8: Optional[torch.Tensor] = None,   # block-scaled (mxfp8) Q/K: UE8M0 scale tiles from mxfp8_qk_quant
    k_scale_e8: Optional[torch.Tensor] = None,
    v_kind: str,                    # "fp8_channel" | "fp8_block" | "mxfp8"
    v_scale: torch.Tensor,
    v_block: int = 0,
    sm_scale: float,
    p_max_offset: int,
    block_m: int = 64,
    block_n: int = 64,
    v_alpha: Optional[torch.Tensor] = None,
    v_smooth_block: int = 0,
    qm_corr: Optional[torch.Tensor] = None,       # (B, H, G, corr_stride) fp32 from qm_corr()
    q_smooth_block: int = 0,
    p_quant_mode: str = "elementwise",
    p_mx_block_n: int = 0,
    rowmax_est_bhs: Optional[torch.Tensor] = None,
    rowmax_init_bhs: Optional[torch.Tensor] = None,
    blasst_lambda: Optional[float] = None,
    blasst_fill_mode: Optional[str] = "zero",
    blasst_fill_alpha: float = 1.0,
    blasst_uta_bins: int = 16,
    return_blasst_stats: bool = False,
    blasst_tile_predicate: bool = False,
    blasst_elided: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    out_nhd: bool = False,
    out_row_index: Optional[torch.Tensor] = None,
    out_fp32_exact: bool = False,
    rowmax_counters: Optional[torch.Tensor] = None,
):
    """Streaming attention on e4m3 operands; output (B,H,M,D) or NHD (B,M,H,D).

    ``rowmax_counters``: optional int64 tensor of 6 zeros on the device; the kernel adds its row-max update
    counts to it (see ``low_bit_fake_quant.diagnostics``).

    ``out_row_index`` (B*H, M) int64 scatters kernel row r to output row
    ``out_row_index[bh, r]`` (the inverse Q reorder fused into the store).

    ``blasst_tile_predicate``: a key block is dropped only when every row of the 128-row tile finds it under the
    threshold, and then for the whole tile (the predicate of the reference's simulator, blasst_skip.py:573-585) instead
    of row by row; zero fill only. ``blasst_elided``: optional int64 tensor of one zero on the device; the kernel adds
    the number of (128-row tile, key block) pairs it did no softmax and no P.V for.
    """
    if not q_codes.is_cuda:
        raise ValueError("operands must live on CUDA")
    B, H, m_pad, D = q_codes.shape
    n_pad = k_codes.shape[2]
    M, N = int(seq_q), int(seq_k)
    dev = q_codes.device
    if p_quant_mode not in L.P_KINDS:
        raise ValueError(f"unknown p_quant_mode: {p_quant_mode!r}")
    if p_quant_mode == "mx":
        if p_mx_block_n <= 0:
            raise ValueError("p_mx_block_n must be > 0 when p_quant_mode='mx'")
        if p_mx_block_n != block_n:
            raise ValueError(
                f"p_mx_block_n ({p_mx_block_n}) currently must equal block_n ({block_n}); "
                "sub-block scaling within a K block is not implemented")
    use_blasst = blasst_lambda is not None
    if use_blasst:
        if not (0.0 < float(blasst_lambda) < 1.0):
            raise ValueError(f"blasst_lambda must be in (0, 1); got {blasst_lambda}")
        fill_kind, fill_alpha, uta_bins = _parse_blasst_fill(
            blasst_fill_mode, alpha=blasst_fill_alpha, uta_bins=blasst_uta_bins)
        if fill_kind == _BLASST_FILL_UTA and block_n % uta_bins != 0:
            raise ValueError(f"blasst UTA bins ({uta_bins}) must divide block_n ({block_n})")
    else:
        if blasst_fill_mode not in ("zero", None):
            raise ValueError("blasst_fill_mode requires blasst_lambda")
        fill_kind, fill_alpha, uta_bins = _BLASST_FILL_ZERO, 1.0, 1
    if blasst_tile_predicate:
        if not use_blasst:
            raise ValueError("blasst_tile_predicate requires blasst_lambda")
        if fill_kind != _BLASST_FILL_ZERO:
            raise ValueError("blasst_tile_predicate drops whole tiles: only the zero fill applies")
        if rowmax_init_bhs is not None:
            raise ValueError("blasst_tile_predicate is built for the online row max without rowmax_init_bhs")
    if blasst_elided is not None and (blasst_elided.dtype != torch.int64 or blasst_elided.numel() != 1
                                      or blasst_elided.device != q_codes.device):
        raise ValueError("blasst_elided must be one int64 value on the operands' device")
    if rowmax_est_bhs is not None and rowmax_init_bhs is not None:
        raise ValueError("rowmax_init_bhs and rowmax_est_bhs are mutually exclusive")
    v_kind_code = {"fp8_channel": L.V_CHANNEL, "fp8_block": L.V_BLOCK, "mxfp8": L.V_MX}[v_kind]

    keep = []   # tensors that must outlive the launch call

    def f32(t):
        if t is None:
            return None
        t = t.to(torch.float32).contiguous()
        keep.append(t)
        return t

    q_scale, k_scale, v_scale = f32(q_scale), f32(k_scale), f32(v_scale)
    v_alpha, qm_corr = f32(v_alpha), f32(qm_corr)
    rowmax_est_bhs, rowmax_init_bhs = f32(rowmax_est_bhs), f32(rowmax_init_bhs)

    stats = None
    if return_blasst_stats:
        stats = torch.zeros(((M + block_m - 1) // block_m, B * H, 2), dtype=torch.float32, device=dev)
    out_shape = (B, M, H, D) if out_nhd else (B, H, M, D)
    out = torch.empty(out_shape, dtype=out_dtype, device=dev)

    with torch.cuda.device(dev):
        status = _status_for(dev)
        a = L.AttnArgs()
        a.B, a.H, a.M, a.N, a.D = B, H, M, N, D
        a.m_pad, a.n_pad = m_pad, n_pad
        a.q_codes, a.k_codes, a.v_codes = q_codes.data_ptr(), k_codes.data_ptr(), v_codes_t.data_ptr()
        a.qk_kind = (L.QK_BF16_V_CODES if qk_bf16_v_codes else L.QK_BF16 if operands_bf16
                     else (L.QK_MX if q_scale_e8 is not None else L.QK_FP8_BLOCK))
        a.q_scale, a.k_scale, a.qk_block = L.ptr(q_scale), L.ptr(k_scale), int(qk_block)
        a.q_scale_e8, a.k_scale_e8 = L.ptr(q_scale_e8), L.ptr(k_scale_e8)
        a.v_kind, a.v_scale, a.v_block = v_kind_code, L.ptr(v_scale), int(v_block)
        a.sm_scale, a.p_max_offset = float(sm_scale), float(p_max_offset)
        a.p_kind = L.P_KINDS[p_quant_mode]
        a.block_m, a.block_n = int(block_m), int(block_n)
        a.v_alpha, a.v_smooth_block = L.ptr(v_alpha), int(v_smooth_block)
        a.qm_corr, a.q_smooth_block = L.ptr(qm_corr), int(q_smooth_block)
        a.corr_stride = int(qm_corr.shape[-1]) if qm_corr is not None else 0
        a.rowmax_est, a.rowmax_init = L.ptr(rowmax_est_bhs), L.ptr(rowmax_init_bhs)
        a.use_blasst = 1 if use_blasst else 0
        a.blasst_lambda = float(blasst_lambda) if use_blasst else 0.0
        a.fill_kind, a.fill_alpha, a.uta_bins = int(fill_kind), float(fill_alpha), int(uta_bins)
        a.blasst_stats = L.ptr(stats)
        a.blasst_tile_predicate = 1 if blasst_tile_predicate else 0
        a.blasst_elided = L.ptr(blasst_elided)
        a.out = out.data_ptr()
        a.out_dtype = L.dtype_code(out_dtype)
        a.out_layout = L.LAYOUT_NHD if out_nhd else L.LAYOUT_BHSD
        a.out_row_index = L.ptr(out_row_index.contiguous()) if out_row_index is not None else None
        a.out_fp32_exact = 1 if out_fp32_exact else 0
        a.status = status.data_ptr()
        if rowmax_counters is not None:
            if rowmax_counters.dtype != torch.int64 or rowmax_counters.numel() != 6 or rowmax_counters.device != dev:
                raise ValueError("rowmax_counters must be 6 int64 values on the operands' device")
            a.rowmax_counters = rowmax_counters.data_ptr()
        ws_bytes = L.lib().lbfq_attention_workspace_bytes(C.byref(a))
        ws = torch.empty((max(int(ws_bytes), 1),), dtype=torch.uint8, device=dev)
        if KERNEL_EVENTS is not None:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        L.check(L.lib().lbfq_attention_fwd(C.byref(a), ws.data_ptr(), L.stream_ptr(dev)))
        if KERNEL_EVENTS is not None:
            ev1.record()
            KERNEL_EVENTS.append((ev0, ev1))
        L.fetch_status(dev)
    if return_blasst_stats:
        return out, stats
    return out


def qm_corr(qm: torch.Tensor, k_smooth: torch.Tensor, *, sm_scale: float, s_pad: int,
            want_rowmax: bool = False):
    """``corr[b,h,g,n] = (qm[b,g,h,:] . k_smooth[b,n,h,:]) * sm_scale`` (fp32, (B,H,G,s_pad))
    and optionally its row max (B,H,G) -- the Q-smoothing score correction of
    attention_triton.py:156-160 and the estimate of attention.py:366-395."""
    b, g, h, d = qm.shape
    _, s, hk, dk = k_smooth.shape
    if h != hk or d != dk:
        raise ValueError(f"qm/k shape mismatch: qm={tuple(qm.shape)} k={tuple(k_smooth.shape)}")
    qm = qm.to(torch.float32).contiguous()
    k_smooth = k_smooth.contiguous()
    corr = torch.empty((b, h, g, s_pad), dtype=torch.float32, device=qm.device)
    rowmax = torch.empty((b, h, g), dtype=torch.float32, device=qm.device) if want_rowmax else None
    with torch.cuda.device(qm.device):
        status = L.status_for(qm.device)
        L.check(L.lib().lbfq_qm_corr(qm.data_ptr(), k_smooth.data_ptr(), L.dtype_code(k_smooth.dtype), b, s, h, d, g,
                                     float(sm_scale), corr.data_ptr(), s_pad, L.ptr(rowmax), status.data_ptr(),
                                     L.stream_ptr(qm.device)))
        L.fetch_status(qm.device)
    return corr, rowmax


__all__ = ["fake_quant_attention_fp8", "fake_quant_attention_triton", "qm_corr", "raise_if_device_error"]


def fake_quant_attention_triton(
    q_bhsd: torch.Tensor,
    k_bhsd: torch.Tensor,
    v_bhsd_bf16: torch.Tensor,
    v_scale_bhd: torch.Tensor,
    *,
    sm_scale: float,
    p_max_offset: int,
    block_m: int = 64,
    block_n: int = 64,
    v_alpha: Optional[torch.Tensor] = None,
    v_smooth_block: int = 0,
    k_smooth_bhsd: Optional[torch.Tensor] = None,
    qm_bhgd: Optional[torch.Tensor] = None,
    q_smooth_block: int = 0,
    v_block_scale_bsh: Optional[torch.Tensor] = None,
    v_block_size: int = 0,
    p_quant_mode: str = "elementwise",
    p_mx_block_n: int = 0,
    rowmax_est_bhs: Optional[torch.Tensor] = None,
    rowmax_init_bhs: Optional[torch.Tensor] = None,
    blasst_lambda: Optional[float] = None,
    blasst_fill_mode: str = "zero",
    blasst_fill_alpha: float = 1.0,
    blasst_uta_bins: int = 16,
    return_blasst_stats: bool = False,
    _out_fp32: bool = False,
    _corr: Optional[torch.Tensor] = None,
):
    """The reference's direct-launch entry (src/low_bit_fake_quant/attention_triton.py:410-671), same signature.

    ``q_bhsd`` / ``k_bhsd``: the de-quantised BF16 operands (B, H, S, D); ``v_bhsd_bf16``: V as BF16 (code values or
    pre-de-quantised) with its per-channel post-scale ``v_scale_bhd`` (FP32 ones when unused). Returns (B, H, S, D)
    BF16, and the stats tensor (ceil(S / block_m), B * H, 2) with ``return_blasst_stats``.

    Two kernels serve it. Without BLASST and without a per-block V scale, Q.K^T and P.V run as BF16 MMAs on exactly
    these operands with the accumulator in tensor memory. With ``v_block_scale_bsh`` (fp8_block V), ``blasst_lambda``
    or ``return_blasst_stats`` the general kernel takes over: Q.K^T is still a BF16 MMA on the given Q / K, V goes back
    to the e4m3 codes it came from (the cast is checked to be exact; a pre-de-quantised mxfp8 V is re-quantised in
    blocks of ``block_n`` keys, which is exact too) and P.V is an FP8 MMA with the V scale, the P scale and the
    V-smoothing term applied in FP32 around it.
    """
    if q_bhsd.ndim != 4 or k_bhsd.shape[:2] != q_bhsd.shape[:2] or v_bhsd_bf16.shape != k_bhsd.shape:
        raise ValueError("q/k/v must be (B, H, S, D) with matching batch, heads and key length")
    for t in (q_bhsd, k_bhsd, v_bhsd_bf16):
        if t.dtype != torch.bfloat16:
            raise TypeError("q_bhsd, k_bhsd and v_bhsd_bf16 must be BF16")
    if v_scale_bhd.dtype != torch.float32:
        raise TypeError("v_scale_bhd must be FP32")
    if blasst_lambda is None and blasst_fill_mode not in ("zero", None):
        raise ValueError("blasst_fill_mode requires blasst_lambda")
    B, H, M, D = q_bhsd.shape
    N = k_bhsd.shape[2]
    if v_scale_bhd.shape != (B, H, D):
        raise ValueError("v_scale_bhd must be (B, H, D)")
    if v_alpha is not None:
        if v_smooth_block <= 0:
            raise ValueError("v_smooth_block must be > 0 when v_alpha is given")
        if v_smooth_block < block_n or v_smooth_block % block_n != 0:
            raise ValueError(f"v_smooth_block ({v_smooth_block}) must be >= block_n ({block_n}) "
                             "and an integer multiple of block_n")
        if N % v_smooth_block != 0:
            raise ValueError(f"S ({N}) must be divisible by v_smooth_block ({v_smooth_block})")
    corr = None
    m_pad, n_pad = (M + 127) // 128 * 128, (N + 127) // 128 * 128
    if qm_bhgd is not None:
        if k_smooth_bhsd is None:
            raise ValueError("k_smooth_bhsd required with qm_bhgd")
        if q_smooth_block <= 0:
            raise ValueError("q_smooth_block must be > 0 with qm_bhgd")
        if q_smooth_block < block_m or q_smooth_block % block_m != 0:
            raise ValueError(f"q_smooth_block ({q_smooth_block}) must be >= block_m ({block_m}) "
                             "and an integer multiple of block_m")
        if M % q_smooth_block != 0:
            raise ValueError(f"S ({M}) must be divisible by q_smooth_block ({q_smooth_block})")
        # despite its name the reference takes this tensor as group_mean_q returns it: (B, S / q_smooth_block, H, D)
        # (attention_triton.py:511)
        n_groups = M // q_smooth_block
        if tuple(qm_bhgd.shape) != (B, n_groups, H, D):
            raise ValueError(f"qm_bhgd must be (B, S // q_smooth_block, H, D) = {(B, n_groups, H, D)}; got {tuple(qm_bhgd.shape)}")
        if tuple(k_smooth_bhsd.shape) != (B, H, N, D):
            raise ValueError(f"k_smooth_bhsd must be {(B, H, N, D)}; got {tuple(k_smooth_bhsd.shape)}")
        if _corr is not None and tuple(_corr.shape) == (B, H, n_groups, n_pad):
            corr = _corr                                  # the caller has formed the product already
        else:
            corr, _ = qm_corr(qm_bhgd.float().contiguous(), k_smooth_bhsd.permute(0, 2, 1, 3).contiguous(),
                              sm_scale=sm_scale, s_pad=n_pad, want_rowmax=False)

    def pad_rows(t, rows):       # (B, H, S, D) -> (B, H, rows, D), zero rows appended
        if t.shape[2] == rows:
            return t.contiguous()
        out = t.new_zeros(t.shape[0], t.shape[1], rows, t.shape[3])
        out[:, :, : t.shape[2]] = t
        return out

    q_p, k_p = pad_rows(q_bhsd, m_pad), pad_rows(k_bhsd, n_pad)
    if v_block_scale_bsh is not None or blasst_lambda is not None or return_blasst_stats:
        # ---- the general kernel: V as e4m3 codes again ----
        if v_block_scale_bsh is not None:
            if v_block_size <= 0:
                raise ValueError("v_block_size must be > 0 when v_block_scale_bsh is given")
            if v_block_size < block_n or v_block_size % block_n != 0:
                raise ValueError(f"v_block_size ({v_block_size}) must be >= block_n ({block_n}) "
                                 "and an integer multiple of block_n")
            if N % v_block_size != 0:
                raise ValueError(f"S ({N}) must be divisible by v_block_size ({v_block_size})")
            if tuple(v_block_scale_bsh.shape) != (B, N // v_block_size, H) or v_block_scale_bsh.dtype != torch.float32:
                raise ValueError(f"v_block_scale_bsh must be FP32 {(B, N // v_block_size, H)}")
        codes = v_bhsd_bf16.to(torch.float8_e4m3fn)
        exact = bool((codes.to(torch.bfloat16) == v_bhsd_bf16).all())
        if v_block_scale_bsh is not None:
            if not exact:
                raise ValueError("with v_block_scale_bsh, v_bhsd_bf16 must hold e4m3 code values (FP8 cast to BF16)")
            v_kind, v_scale, v_blk = "fp8_block", v_block_scale_bsh, v_block_size
        elif exact:
            v_kind, v_scale, v_blk = "fp8_channel", v_scale_bhd, 0
        else:
            # a pre-de-quantised mxfp8 V (codes x 2^e per channel and key block): re-quantising any sub-block of the
            # original blocks recovers codes and power-of-two scales exactly
            from .quant_triton import mxfp8_v_dequant, mxfp8_v_quant
            if not bool((v_scale_bhd == 1.0).all()) or N % block_n != 0:
                raise NotImplementedError("this V is neither e4m3 code values nor a de-quantised mxfp8 tensor with unit v_scale")
            v_nhd = v_bhsd_bf16.permute(0, 2, 1, 3).contiguous()
            c_nhd, v_scale = mxfp8_v_quant(v_nhd, block_s=block_n)
            if not bool((mxfp8_v_dequant(c_nhd, v_scale, block_s=block_n, dtype=torch.bfloat16) == v_nhd).all()):
                raise NotImplementedError("this V is neither e4m3 code values nor a de-quantised mxfp8 tensor")
            codes = c_nhd.permute(0, 2, 1, 3)
            v_kind, v_blk = "mxfp8", block_n
        v_t = torch.zeros((B, H, D, n_pad), dtype=torch.float8_e4m3fn, device=q_bhsd.device)
        v_t.view(torch.uint8)[..., :N] = codes.contiguous().view(torch.uint8).transpose(2, 3)
        return fake_quant_attention_fp8(
            q_p, k_p, v_t, seq_q=M, seq_k=N, q_scale=None, k_scale=None, qk_block=block_n, qk_bf16_v_codes=True,
            v_kind=v_kind, v_scale=v_scale, v_block=v_blk,
            sm_scale=float(sm_scale), p_max_offset=int(p_max_offset), block_m=block_m, block_n=block_n,
            v_alpha=v_alpha, v_smooth_block=v_smooth_block, qm_corr=corr, q_smooth_block=q_smooth_block,
            p_quant_mode=p_quant_mode, p_mx_block_n=p_mx_block_n,
            rowmax_est_bhs=rowmax_est_bhs, rowmax_init_bhs=rowmax_init_bhs,
            blasst_lambda=blasst_lambda, blasst_fill_mode=blasst_fill_mode, blasst_fill_alpha=blasst_fill_alpha,
            blasst_uta_bins=blasst_uta_bins, return_blasst_stats=return_blasst_stats,
            out_dtype=torch.float32 if _out_fp32 else torch.bfloat16, out_nhd=False, out_fp32_exact=_out_fp32,
        )
    v_t = pad_rows(v_bhsd_bf16, n_pad).transpose(2, 3).contiguous()              # (B, H, D, n_pad), keys contiguous
    return fake_quant_attention_fp8(
        q_p, k_p, v_t, seq_q=M, seq_k=N, q_scale=None, k_scale=None, qk_block=block_n, operands_bf16=True,
        v_kind="fp8_channel", v_scale=v_scale_bhd, v_block=0,
        sm_scale=float(sm_scale), p_max_offset=int(p_max_offset), block_m=block_m, block_n=block_n,
        v_alpha=v_alpha, v_smooth_block=v_smooth_block, qm_corr=corr, q_smooth_block=q_smooth_block,
        p_quant_mode=p_quant_mode, p_mx_block_n=p_mx_block_n,
        rowmax_est_bhs=rowmax_est_bhs, rowmax_init_bhs=rowmax_init_bhs,
        out_dtype=torch.float32 if _out_fp32 else torch.bfloat16, out_nhd=False, out_fp32_exact=_out_fp32,
    )
