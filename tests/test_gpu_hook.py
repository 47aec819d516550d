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


# --- cross-attention (K / V of their own length): an extension, checked against the oracle's same extension ----------

CROSS = {
    "k_smooth_static": dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, smoothing="k_only", q_kmeans_k=None),
    "mxfp8_hadamard": dict(qk_quant="mxfp8", v_quant="mxfp8", smoothing="off", q_kmeans_k=None, qk_hadamard=True),
    "full_dynamic": dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, q_smooth_block_size=128,
                         smoothing="full", q_kmeans_k=4, v_kmeans_k=4, v_smooth_mode="per_block", p_quant="dynamic",
                         rowmax_mode="qm_k"),
    "blasst": dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, smoothing="k_only", q_kmeans_k=None,
                   p_quant="dynamic", blasst_lambda=1e-1, blasst_fill="mean_a1.5"),
}


@pytest.mark.parametrize("name", sorted(CROSS))
@pytest.mark.parametrize("sq,sk", [(1024, 512), (256, 1536), (640, 192)])
def test_cross_attention_matches_oracle(name, sq, sk):
    from low_bit_fake_quant import _lib as L
    from low_bit_fake_quant.attention import fake_quant_attention
    from low_bit_fake_quant.attention_triton import raise_if_device_error
    from low_bit_fake_quant.hook import fake_quant_cross_attention
    from oracle import api as OA
    cfg = QuantConfig(**CROSS[name])
    torch.manual_seed(sq + sk)
    q = torch.randn(1, sq, 2, 128).bfloat16()
    k = (torch.randn(1, sk, 2, 128) + 1.5 * torch.randn(1, 1, 2, 128)).bfloat16()
    v = torch.randn(1, sk, 2, 128).bfloat16()
    got = fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg, _cross=True, _debug_fp32=True).float().cpu()
    raise_if_device_error(torch.device(DEV))
    p_bf16 = L.lib().lbfq_attention_last_variant() == 1
    ql = vl = None
    if cfg.q_kmeans_k is not None or cfg.v_kmeans_k is not None:      # k-means labels are not pinned: hand over the GPU's
        from low_bit_fake_quant.attention import _preprocess
        pre = _preprocess(q.to(DEV), k.to(DEV), v.to(DEV), cfg)
        ql, vl = pre[5].labels.cpu(), pre[6].labels.cpu()
    want = OA.fake_quant_attention(q, k, v, cfg, faithful=False, out_fp32=True, cross=True, p_bf16=p_bf16,
                                   q_labels=ql, v_labels=vl)
    assert got.shape == q.shape
    assert OA.parity_ok(OA.parity_report(got, want, q, k, v)), OA.parity_report(got, want, q, k, v)
    out = fake_quant_cross_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg)
    assert out.dtype == q.dtype and out.shape == q.shape and torch.isfinite(out).all()


def test_cross_attention_errors():
    from low_bit_fake_quant.hook import fake_quant_cross_attention
    q = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, device=DEV)
    cfg = QuantConfig(qk_quant="fp8_block", fp8_block_size=64, smoothing="off", q_kmeans_k=None)
    with pytest.raises(ValueError, match="cross-attention wants"):
        fake_quant_cross_attention(q, k, k[:, :64], cfg)
    with pytest.raises(ValueError, match="p_requant=True"):
        fake_quant_cross_attention(q, k, k, QuantConfig(qk_quant="fp8_block", fp8_block_size=64, smoothing="off",
                                                        q_kmeans_k=None, p_requant=False))
    with pytest.raises(ValueError, match="shapes must match"):
        fq.fake_quant_attention(q, k, k, cfg)                 # the reference's entry keeps its equal-shape rule


def test_reordered_entry_is_a_permutation_round_trip():
    """Tokens taken brick by brick (bench/eval_blasst_quant.py:101-134 of the reference), result back in the original
    order: equal to permuting by hand, and as close to full-precision attention as the plain call."""
    from low_bit_fake_quant.hook import fake_quant_attention_reordered, space_time_block_order
    cfg = QuantConfig(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, smoothing="k_only", q_kmeans_k=None,
                      p_quant="dynamic", blasst_lambda=1e-2, blasst_fill="mean_a1.5")
    torch.manual_seed(6)
    t, h, w = 4, 8, 16                                   # 512 tokens
    q, k, v = (torch.randn(1, t * h * w, 2, 128, device=DEV).bfloat16() for _ in range(3))
    order = space_time_block_order(t, h, w, ts=2, hs=4, ws=8, device=DEV)
    got = fake_quant_attention_reordered(q, k, v, cfg, order)
    by_hand = fq.fake_quant_attention(q[:, order].contiguous(), k[:, order].contiguous(), v[:, order].contiguous(), cfg)
    want = torch.empty_like(by_hand)
    want[:, order] = by_hand
    assert torch.equal(got, want)
    ref = fq.reference_attention(q, k, v).float()
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), ref.flatten(), dim=0)
    assert cos > 0.99
    with pytest.raises(ValueError, match="permutation"):
        fake_quant_attention_reordered(q, k, v, cfg, order[:-1])
