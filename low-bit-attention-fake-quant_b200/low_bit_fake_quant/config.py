"""Configuration object of the fake-quant attention path.

Field-for-field mirror of the reference ``QuantConfig``
(src/low_bit_fake_quant/config.py:35-122): same names, same defaults, same
``Literal`` aliases (config.py:8-32), frozen. Code written against the
reference configuration object runs unchanged against this one.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional

import torch

QKQuant = Literal["fp8_block", "mxfp8"]
VQuant = Literal["fp8_channel", "fp8_block", "mxfp8"]
Smoothing = Literal["off", "k_only", "full"]
VSmoothMode = Literal["off", "per_block"]
PQuant = Literal["auto", "elementwise", "mx", "dynamic"]
RowmaxMode = Literal["online", "qm_k"]
# Free-form: "zero", "max", "mean", "logn", "sample8", "thr", "uta" and the
# probe spellings "mean_a1.5", "uta16_a1.5", ... (attention_triton.py:674-714).
BlasstFill = str


@dataclass(frozen=True)
class QuantConfig:
    """Knobs of :func:`low_bit_fake_quant.fake_quant_attention`.

    Quantisation of Q/K (``fp8_block``: one FP32 scale per (B, S/blk, H);
    ``mxfp8``: one power-of-two scale per 32 elements of D), of V
    (``fp8_channel``: per (B, H, D); ``fp8_block``: per (B, S/blk, H);
    ``mxfp8``: power-of-two per (B, S/blk, H, D), blocks along S), of the
    softmax numerator P, plus the accuracy helpers around them (K / Q / V
    smoothing, Hadamard rotation, k-means token reorder, estimated row max,
    BLASST skip/fill).
    """

    qk_quant: QKQuant = "fp8_block"
    v_quant: VQuant = "fp8_channel"
    smoothing: Smoothing = "full"
    q_smooth_block_size: int = 256
    q_kmeans_k: Optional[int] = 32
    q_kmeans_iters: int = 10
    q_kmeans_seed: int = 0
    qk_hadamard: bool = False
    qk_hadamard_random_sign: bool = True
    qk_hadamard_seed: int = 0
    fp8_block_size: int = 128
    mxfp8_block_size: int = 32
    v_fp8_block_size: int = 64
    v_mxfp8_block_size: int = 64
    p_quant: PQuant = "auto"
    rowmax_mode: RowmaxMode = "online"
    p_mx_block_n: int = 0
    p_max_offset: int = 8
    correction_dtype: torch.dtype = torch.float16
    p_requant: bool = True
    p_requant_q_chunk: int = 512
    p_requant_block_m: int = 64
    p_requant_block_n: int = 64
    blasst_lambda: Optional[float] = None
    blasst_fill: BlasstFill = "zero"
    blasst_fill_alpha: float = 1.0
    blasst_uta_bins: int = 16
    v_smooth_mode: VSmoothMode = "off"
    v_smooth_block_size: int = 64
    v_kmeans_k: Optional[int] = None
    v_kmeans_iters: int = 10
    v_kmeans_seed: int = 0
