"""ctypes binding of ``liblbfq.so`` (the sm_100a CUDA library) -- plumbing only.

The library is looked up next to the package (``../liblbfq.so``, built by
``build.sh``). There is no fallback: if it is missing, importing any op of this
package raises, and every op refuses CPU tensors exactly as the reference does.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LBFQ_LIB", os.path.join(os.path.dirname(_HERE), "liblbfq.so"))

F32, F16, BF16 = 0, 1, 2
LAYOUT_NHD, LAYOUT_BHSD, LAYOUT_BHDS = 0, 1, 2
P_KINDS = {"elementwise": 0, "mx": 1, "dynamic": 2}
V_CHANNEL, V_BLOCK, V_MX = 0, 1, 2
QK_FP8_BLOCK, QK_MX, QK_BF16, QK_BF16_V_CODES = 0, 1, 2, 3

ERR_ARG, ERR_DTYPE, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE = -1, -2, -3, -4, -5
# debug overrides (LBFQ_FLAG_* of include/lbfq.h)
FLAG_ATTN_GENERIC, FLAG_KMEANS_FFMA, FLAG_QM_CORR_FFMA, FLAG_UNFUSED_PREPROCESS, FLAG_KMEANS_SORTED = 1, 2, 4, 8, 16

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


class AttnArgs(C.Structure):
    """Mirror of ``lbfq_attn_args`` (include/lbfq.h)."""

    _fields_ = [
        ("B", C.c_int), ("H", C.c_int), ("M", C.c_int), ("N", C.c_int), ("D", C.c_int),
        ("m_pad", C.c_int), ("n_pad", C.c_int),
        ("q_codes", C.c_void_p), ("k_codes", C.c_void_p), ("v_codes", C.c_void_p),
        ("qk_kind", C.c_int),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p),
        ("qk_block", C.c_int),
        ("q_scale_e8", C.c_void_p), ("k_scale_e8", C.c_void_p),
        ("v_kind", C.c_int),
        ("v_scale", C.c_void_p),
        ("v_block", C.c_int),
        ("sm_scale", C.c_float), ("p_max_offset", C.c_float),
        ("p_kind", C.c_int),
        ("block_m", C.c_int), ("block_n", C.c_int),
        ("v_alpha", C.c_void_p),
        ("v_smooth_block", C.c_int),
        ("qm_corr", C.c_void_p),
        ("q_smooth_block", C.c_int),
        ("corr_stride", C.c_int),
        ("rowmax_est", C.c_void_p), ("rowmax_init", C.c_void_p),
        ("use_blasst", C.c_int),
        ("blasst_lambda", C.c_float),
        ("fill_kind", C.c_int),
        ("fill_alpha", C.c_float),
        ("uta_bins", C.c_int),
        ("blasst_stats", C.c_void_p),
        ("blasst_tile_predicate", C.c_int),
        ("blasst_elided", C.c_void_p),
        ("out", C.c_void_p),
        ("out_dtype", C.c_int), ("out_layout", C.c_int),
        ("out_row_index", C.c_void_p),
        ("out_fp32_exact", C.c_int),
        ("status", C.c_void_p),
        ("rowmax_counters", C.c_void_p),
    ]


class PrepArgs(C.Structure):
    """Mirror of ``lbfq_prep_args`` (include/lbfq.h)."""

    _fields_ = [
        ("x", C.c_void_p), ("dtype", C.c_int),
        ("B", C.c_int), ("S", C.c_int), ("H", C.c_int), ("D", C.c_int),
        ("order", C.c_void_p), ("chan_mean", C.c_void_p),
        ("smooth_block", C.c_int), ("block_mean", C.c_void_p),
        ("hadamard", C.c_int), ("signs", C.c_void_p), ("had_scale", C.c_float),
        ("kind", C.c_int), ("scale_block", C.c_int),
        ("codes", C.c_void_p), ("layout", C.c_int), ("s_pad", C.c_int),
        ("scale", C.c_void_p), ("scale_e8", C.c_void_p), ("smooth_out", C.c_void_p),
    ]


PREP_FP8_BLOCK, PREP_FP8_CHANNEL, PREP_MXFP8_V, PREP_MXFP8_QK = 0, 1, 2, 3

_P = C.c_void_p
_I = C.c_int
_SIGS = {
    "lbfq_last_error": (C.c_char_p, []),
    "lbfq_abi_version": (_I, []),
    "lbfq_launch_count": (C.c_ulonglong, []),
    "lbfq_get_flags": (_I, []),
    "lbfq_set_flags": (None, [_I]),
    "lbfq_attention_last_variant": (_I, []),
    "lbfq_rcp_approx": (_I, [_P, _P, C.c_longlong, _P]),
    "lbfq_copy_rows_async": (_I, [_P, C.c_size_t, _P, C.c_size_t, C.c_size_t, C.c_size_t, _I, _P]),
    "lbfq_fp8_block_quant": (_I, [_P, _I, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P]),
    "lbfq_fp8_block_quant_centered": (_I, [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P, _P]),
    "lbfq_fp8_block_dequant": (_I, [_P, _P, _I, _I, _I, _I, _I, _P, _I, _P]),
    "lbfq_fp8_channel_quant": (_I, [_P, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P]),
    "lbfq_fp8_channel_dequant": (_I, [_P, _P, _I, _I, _I, _I, _P, _I, _P]),
    "lbfq_mxfp8_qk_quant": (_I, [_P, _I, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P]),
    "lbfq_mxfp8_qk_dequant": (_I, [_P, _P, _I, _I, _I, _I, _I, _P, _I, _P]),
    "lbfq_mxfp8_v_quant": (_I, [_P, _I, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P]),
    "lbfq_mxfp8_v_dequant": (_I, [_P, _P, _I, _I, _I, _I, _I, _P, _I, _P]),
    "lbfq_prep_group_rows": (_I, [_I, _I, _I, _I, _I, _I]),
    "lbfq_prep_fused": (_I, [C.POINTER(PrepArgs), _P]),
    "lbfq_smooth_k_scratch_floats": (C.c_int64, [_I, _I, _I, _I]),
    "lbfq_smooth_k": (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P, _P]),
    "lbfq_smooth_k_static_max_floats": (C.c_int64, []),
    "lbfq_smooth_k_static": (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P]),
    "lbfq_block_mean_sub": (_I, [_P, _I, _I, _I, _I, _I, _I, _P, _P, _P]),
    "lbfq_hadamard": (_I, [_P, _I, C.c_int64, _I, _I, _P, C.c_float, _P, _P]),
    "lbfq_kmeans_scratch_bytes": (C.c_int64, [_I, _I, _I, _I, _I]),
    "lbfq_kmeans_labels": (_I, [_P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P]),
    "lbfq_label_order": (_I, [_P, _I, _I, _I, _P, _P, _P]),
    "lbfq_gather_rows": (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P]),
    "lbfq_qm_corr": (_I, [_P, _P, _I, _I, _I, _I, _I, _I, C.c_float, _P, _I, _P, _P, _P]),
    "lbfq_attention_workspace_bytes": (C.c_int64, [C.POINTER(AttnArgs)]),
    "lbfq_attention_fwd": (_I, [C.POINTER(AttnArgs), _P, _P]),
}

_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """The loaded library; raises ``RuntimeError`` when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build the CUDA library first "
                "(low-bit-attention-fake-quant_b200/build.sh); there is no CPU or Triton fallback")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def exported_symbols():
    return list(_SIGS.keys())


def dtype_code(dt: torch.dtype) -> int:
    if dt not in _DTYPES:
        raise TypeError(f"unsupported dtype {dt}")
    return _DTYPES[dt]


def check(rc: int) -> None:
    """Map a status code to the exception class the reference raises."""
    if rc == 0:
        return
    msg = lib().lbfq_last_error().decode("utf-8", "replace")
    if rc == ERR_ARG:
        raise ValueError(msg)
    if rc == ERR_DTYPE:
        raise TypeError(msg)
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"liblbfq error {rc}: {msg}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# ---------------------------------------------------------------------------
# debug overrides
# ---------------------------------------------------------------------------

def flags() -> int:
    """The library's debug overrides (``FLAG_*``); initialised from the ``LBFQ_*`` environment variables once."""
    return int(lib().lbfq_get_flags())


def set_flag(flag: int, on: bool) -> None:
    """Switch one debug override on or off (process-wide)."""
    cur = flags()
    lib().lbfq_set_flags((cur | flag) if on else (cur & ~flag))


class override:
    """Context manager that switches debug overrides on (``override(FLAG_ATTN_GENERIC)``) for the enclosed calls and
    restores the previous set afterwards. Process-wide: meant for tests and measurements, not for concurrent use."""

    def __init__(self, on: int = 0, off: int = 0):
        self.on, self.off = int(on), int(off)

    def __enter__(self):
        self.saved = flags()
        lib().lbfq_set_flags((self.saved | self.on) & ~self.off)
        return self

    def __exit__(self, *exc):
        lib().lbfq_set_flags(self.saved)
        return False


# ---------------------------------------------------------------------------
# device status word: kernels with bounded waits raise it instead of hanging
# ---------------------------------------------------------------------------

_status_dev: dict[int, torch.Tensor] = {}
_status_host: dict[int, torch.Tensor] = {}


def status_for(device: torch.device) -> torch.Tensor:
    """The int32 status word of ``device`` (created on first use). Raises ``RuntimeError`` if an earlier launch on
    that device reported an expired wait (the word is read back asynchronously after every launch that takes it)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_dev:
        _status_dev[idx] = torch.zeros(1, dtype=torch.int32, device=device)
        _status_host[idx] = torch.zeros(1, dtype=torch.int32).pin_memory()
    host = _status_host[idx]
    if int(host[0]) != 0:
        code = int(host[0])
        host.zero_()
        _status_dev[idx].zero_()
        raise RuntimeError(f"a kernel of liblbfq gave up a bounded wait (code {code}); its results are invalid")
    return _status_dev[idx]


def fetch_status(device: torch.device) -> None:
    """Enqueue the copy of the device's status word to its pinned host mirror (no synchronisation)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _status_dev:
        _status_host[idx].copy_(_status_dev[idx], non_blocking=True)


def raise_if_device_error(device: Optional[torch.device] = None) -> None:
    """Synchronise ``device`` and raise if any launch on it reported an expired wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    torch.cuda.synchronize(device)
    status_for(device)


def rcp_approx(x: torch.Tensor, device: Optional[torch.device] = None) -> torch.Tensor:
    """Element-wise ``rcp.approx.f32`` of an FP32 tensor, computed on the GPU and returned on ``x``'s device: the
    reciprocal the quantizers multiply by. A utility for CPU restatements of the path (see ``lbfq_rcp_approx``)."""
    dev = x.device if x.is_cuda else (torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device()))
    xd = x.detach().to(device=dev, dtype=torch.float32).contiguous()
    yd = torch.empty_like(xd)
    with torch.cuda.device(dev):
        check(lib().lbfq_rcp_approx(xd.data_ptr(), yd.data_ptr(), xd.numel(), stream_ptr(dev)))
    return yd.to(x.device)
