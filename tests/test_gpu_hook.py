"""The padded entry follows the reference hook's policy (bench/wan_attention_hook.py:253-294): S is padded to the
lcm of the block sizes, Q rows with zeros, K / V rows with the last token; the padded rows are dropped."""
import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant.config import QuantConfig
from low_bit_fake_quant.hook import fake_quant_attention_padded, pad_qkv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("kw", [
    dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, smoothing="k_only", q_kmeans_k=None),
    dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=128, smoothing="full", q_smooth_block_size=256,
         q_kmeans_k=8, p_quant="dynamic"),
])
def test_padded_entry_equals_manual_pad_and_slice(kw):
    cfg = QuantConfig(**kw)
    torch.manual_seed(3)
    q, k, v = (torch.randn(1, 1000, 2, 128, device=DEV).bfloat16() for _ in range(3))
    got = fake_quant_attention_padded(q, k, v, cfg, sm_scale=0.1)
    qp, kp, vp, pad = pad_qkv(q, k, v, cfg)
    assert pad > 0 and qp.shape[1] % 64 == 0
    want = fq.fake_quant_attention(qp.contiguous(), kp.contiguous(), vp.contiguous(), cfg, sm_scale=0.1)[:, :1000]
    assert got.shape == q.shape and got.is_contiguous() and torch.equal(got, want)
    # and it is the quantised form of full-precision attention over the same padded keys
    ref = fq.reference_attention(qp.contiguous(), kp.contiguous(), vp.contiguous(), sm_scale=0.1)[:, :1000].float()
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), ref.flatten(), dim=0)
    assert cos > 0.99


def test_padded_entry_is_the_plain_call_when_s_divides():
    cfg = QuantConfig(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, smoothing="k_only", q_kmeans_k=None)
    torch.manual_seed(4)
    q, k, v = (torch.randn(1, 512, 2, 64, device=DEV).bfloat16() for _ in range(3))
    assert torch.equal(fake_quant_attention_padded(q, k, v, cfg), fq.fake_quant_attention(q, k, v, cfg))
