"""B200-native drop-in for the ``low_bit_fake_quant`` package.

Exports the same names as the reference package
(src/low_bit_fake_quant/__init__.py:3-60). Every device step runs in
``liblbfq.so`` (hand-written sm_100a CUDA behind a C ABI, see include/lbfq.h);
there is no Triton, no CPU fallback and no other backend.
"""

from .attention import (
    FakeQuantArtifacts,
    PreprocessCache,
    fake_quant_attention,
    prepare_for_attention,
    reference_attention,
)
from .config import QuantConfig
from .host import fake_quant_attention_host  # extension: not in the reference, hence not in __all__
from .hadamard import apply_qk_hadamard, fast_hadamard_available, hadamard_transform_last_dim
from .kmeans import (
    KMeansReorderResult,
    apply_kv_permutation,
    kmeans_reorder_tokens,
    q_kmeans_reorder,
    v_kmeans_reorder,
)
from .pipeline import PreparedQKV, prepare_qkv
from .preprocess import group_mean_q, smooth_k, smooth_v_per_block
from .quant_triton import (
    fp8_block_dequant,
    fp8_block_quant,
    fp8_per_channel_dequant,
    fp8_per_channel_quant,
    mxfp8_qk_dequant,
    mxfp8_qk_quant,
    mxfp8_v_dequant,
    mxfp8_v_quant,
)

__all__ = [
    "FakeQuantArtifacts",
    "KMeansReorderResult",
    "PreparedQKV",
    "PreprocessCache",
    "QuantConfig",
    "apply_qk_hadamard",
    "fake_quant_attention",
    "fast_hadamard_available",
    "prepare_for_attention",
    "fp8_block_dequant",
    "fp8_block_quant",
    "fp8_per_channel_dequant",
    "fp8_per_channel_quant",
    "group_mean_q",
    "hadamard_transform_last_dim",
    "smooth_v_per_block",
    "mxfp8_qk_dequant",
    "mxfp8_qk_quant",
    "mxfp8_v_dequant",
    "mxfp8_v_quant",
    "prepare_qkv",
    "apply_kv_permutation",
    "kmeans_reorder_tokens",
    "q_kmeans_reorder",
    "v_kmeans_reorder",
    "reference_attention",
    "smooth_k",
]
