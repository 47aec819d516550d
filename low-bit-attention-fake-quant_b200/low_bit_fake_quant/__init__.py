"""B200-native drop-in for the ``low_bit_fake_quant`` package.

The public names are those of the reference package (src/low_bit_fake_quant/__init__.py:3-60); every device step
behind them runs in ``liblbfq.so`` (hand-written sm_100a CUDA behind a C ABI, see include/lbfq.h). There is no
Triton, no CPU fallback and no other backend. ``fake_quant_attention_host`` (host-resident tensors,
copies pipelined with compute) and ``fake_quant_attention_padded`` (the reference hook's pad-to-block-multiple policy)
are extensions and are therefore kept out of ``__all__``.
"""
from . import attention as _attention
from . import hadamard as _hadamard
from . import kmeans as _kmeans
from . import pipeline as _pipeline
from . import preprocess as _preprocess
from . import quant_triton as _quant
from .config import QuantConfig
from .hook import fake_quant_attention_padded
from .host import fake_quant_attention_host

# name -> module that defines it; the export list below is generated from this table
_EXPORTS = {
    _attention: "FakeQuantArtifacts PreprocessCache fake_quant_attention prepare_for_attention reference_attention",
    _hadamard: "apply_qk_hadamard fast_hadamard_available hadamard_transform_last_dim",
    _kmeans: "KMeansReorderResult apply_kv_permutation kmeans_reorder_tokens q_kmeans_reorder v_kmeans_reorder",
    _pipeline: "PreparedQKV prepare_qkv",
    _preprocess: "group_mean_q smooth_k smooth_v_per_block",
    _quant: ("fp8_block_quant fp8_block_dequant fp8_per_channel_quant fp8_per_channel_dequant "
             "mxfp8_qk_quant mxfp8_qk_dequant mxfp8_v_quant mxfp8_v_dequant"),
}
__all__ = ["QuantConfig"]
for _module, _names in _EXPORTS.items():
    for _name in _names.split():
        globals()[_name] = getattr(_module, _name)
        __all__.append(_name)
__all__.sort()
del _module, _names, _name
