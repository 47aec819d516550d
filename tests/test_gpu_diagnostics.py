"""Row-max update counters: the kernel's opt-in epilogue against the oracle's count of the same events
(what bench/count_rowmax_updates_triton.py of the reference measures with a kernel of its own)."""
import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant.attention_triton import raise_if_device_error
from low_bit_fake_quant.config import QuantConfig
from low_bit_fake_quant.diagnostics import COUNTER_NAMES, count_rowmax_updates
from oracle import api as OA

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BASE = dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, q_smooth_block_size=128, q_kmeans_k=None)


def _qkv(seed, B=1, S=1024, H=2, D=128):
    torch.manual_seed(seed)
    q, k, v = torch.randn(B, S, H, D), torch.randn(B, S, H, D), torch.randn(B, S, H, D)
    q[..., :4] *= 4.0
    k[..., :4] *= 4.0
    k = k + 2.0 * torch.randn(1, 1, H, D)
    return q.bfloat16(), k.bfloat16(), v.bfloat16()


@pytest.mark.parametrize("extra", [
    dict(smoothing="k_only"),                                                    # online row max, e4m3 P
    dict(smoothing="full", p_quant="dynamic"),                                   # online, score bias, dynamic P
    dict(smoothing="full", p_quant="dynamic", rowmax_mode="qm_k"),                # estimate + up / down thresholds
    dict(smoothing="full", rowmax_mode="qm_k"),                                  # estimate frozen: no update at all
    dict(smoothing="k_only", blasst_lambda=1e-2),                                 # a skipped row keeps its max
])
def test_counters_match_the_oracle(extra):
    cfg = QuantConfig(**BASE, **extra)
    q, k, v = _qkv(7)
    got = count_rowmax_updates(q.to(DEV), k.to(DEV), v.to(DEV), cfg)
    raise_if_device_error(torch.device(DEV))
    want = {}
    OA.fake_quant_attention(q, k, v, cfg, faithful=False, out_fp32=True, rowmax_counters=want)
    # the scores of the two sides differ in their last bits (summation order), which can flip a near-tie
    for n in COUNTER_NAMES:
        assert abs(got[n] - want[n]) <= 2 + 0.002 * want[n], (n, got, want)
    assert got["upward_updates"] + got["downward_updates"] == got["updates"]
    assert got["rescales"] <= got["updates"] and got["rows_with_update"] <= q.shape[0] * q.shape[1] * q.shape[2]
    if extra.get("rowmax_mode") == "qm_k" and extra.get("p_quant") != "dynamic":
        assert got["updates"] == 0


def test_estimated_row_max_removes_most_rescales():
    """The claim the reference's diagnostic backs (README.md:127-142): with the estimated row max the accumulator is
    rescaled far less often than with the online max."""
    q, k, v = (t.to(DEV) for t in _qkv(8, S=2048))
    kw = dict(BASE, smoothing="full", p_quant="dynamic")
    online = count_rowmax_updates(q, k, v, QuantConfig(**kw))
    est = count_rowmax_updates(q, k, v, QuantConfig(**kw, rowmax_mode="qm_k"))
    assert est["rescales"] * 4 < online["rescales"], (est, online)


def test_counters_leave_the_result_alone():
    q, k, v = (t.to(DEV) for t in _qkv(9, S=512))
    cfg = QuantConfig(**BASE, smoothing="k_only")
    count_rowmax_updates(q, k, v, cfg)                     # general kernel with the counting epilogue
    a = fq.fake_quant_attention(q, k, v, cfg)
    assert torch.isfinite(a).all()
    with pytest.raises(ValueError, match="p_requant=True"):
        count_rowmax_updates(q, k, v, QuantConfig(**BASE, smoothing="k_only", p_requant=False))
