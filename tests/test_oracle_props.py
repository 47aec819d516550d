"""Properties of the CPU oracle: edge cases the reference's arithmetic implies."""
import math

import pytest
import torch

from low_bit_fake_quant.config import QuantConfig
from oracle import api as OA
from oracle import quant_ops as OQ


def test_e4m3_cast_saturates_and_rounds_to_even():
    x = torch.tensor([1000.0, 449.0, 464.0, 465.0, -1000.0, 2.0 ** -9, 2.0 ** -10, 0.75 * 2.0 ** -9, 0.0])
    got = OQ.to_e4m3(x).float()
    want = torch.tensor([448.0, 448.0, 448.0, 448.0, -448.0, 2.0 ** -9, 0.0, 2.0 ** -9, 0.0])
    assert torch.equal(got, want)


def test_pow2_scale_is_exact_ceil_log2():
    # amax / 448 exactly a power of two -> that power; one ulp above -> the next one
    for k in (-10, -3, 0, 5):
        amax = torch.tensor([448.0 * 2.0 ** k])
        assert OQ.pow2_scale(amax).item() == 2.0 ** k
        up = torch.nextafter(amax, torch.tensor([float("inf")]))
        assert OQ.pow2_scale(up).item() == 2.0 ** (k + 1)
    # the edge case: amax = 1.75 * 2^k is the largest bf16 mantissa below 2 -> 448 = 1.75 * 256
    assert OQ.pow2_scale(torch.tensor([1.75 * 2.0 ** 3])).item() == 2.0 ** -5
    assert OQ.pow2_scale(torch.tensor([1e-4])).item() == 2.0 ** math.ceil(math.log2(1e-4 / 448.0))


def test_quantizers_roundtrip_and_shapes():
    torch.manual_seed(0)
    x = (torch.randn(2, 128, 3, 64) * 3).bfloat16()
    c, s = OQ.fp8_block_quant(x, 64)
    assert c.dtype == torch.float8_e4m3fn and s.shape == (2, 2, 3)
    assert c.float().abs().max() <= 448
    d = OQ.fp8_block_dequant(c, s, 64)
    assert (d - x.float()).abs().max() <= x.float().abs().max() * 2 ** -3
    c, s = OQ.fp8_per_channel_quant(x)
    assert s.shape == (2, 3, 64) and c.float().abs().amax(dim=1).min() == 448.0   # every channel hits full scale
    c, s = OQ.mxfp8_qk_quant(x, 32)
    assert s.shape == (2, 128, 3, 2) and torch.equal(s, torch.exp2(torch.log2(s).round()))
    assert torch.equal(OQ.mxfp8_qk_dequant(c, s, 32, dtype=torch.bfloat16).float(), c.float().reshape(2, 128, 3, 2, 32).mul(s[..., None]).reshape(2, 128, 3, 64))
    c, s = OQ.mxfp8_v_quant(x, 32)
    assert s.shape == (2, 4, 3, 64)
    with pytest.raises(ValueError):
        OQ.fp8_block_quant(x, 48)
    with pytest.raises(ValueError):
        OQ.fp8_block_quant(torch.zeros(1, 8, 1, 32), 8)


def test_amax_floor_on_zero_input():
    z = torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16)
    c, s = OQ.fp8_block_quant(z, 64)
    assert s.item() == pytest.approx(1e-4 / 448.0) and c.float().abs().sum() == 0


def test_smoothing_means():
    torch.manual_seed(1)
    k = (torch.randn(1, 512, 2, 64) + 3).bfloat16()
    ks, mean = OQ.smooth_k(k)
    assert ks.dtype == k.dtype and mean.shape == (1, 2, 64)
    torch.testing.assert_close(mean, k.float().mean(dim=1), rtol=1e-5, atol=1e-5)
    assert ks.float().mean(dim=1).abs().max() < 1e-2
    v, alpha = OQ.smooth_v_per_block(k, 64)
    assert alpha.shape == (1, 8, 2, 64)
    torch.testing.assert_close(alpha, k.float().reshape(1, 8, 64, 2, 64).mean(dim=2), rtol=1e-5, atol=1e-5)


def test_hadamard_is_orthonormal_and_preserves_logits():
    torch.manual_seed(2)
    q = torch.randn(1, 64, 2, 128)
    k = torch.randn(1, 64, 2, 128)
    qr, kr = OQ.apply_qk_hadamard(q, k, seed=3)
    a = torch.einsum("bshd,bthd->bhst", q, k)
    b = torch.einsum("bshd,bthd->bhst", qr, kr)
    assert (a - b).abs().max() < 2e-4          # the reference's own bound (tests/test_qk_hadamard.py:36)
    torch.testing.assert_close(qr.pow(2).sum(-1), q.pow(2).sum(-1), rtol=1e-5, atol=1e-5)


def test_kmeans_reorder_invariants():
    torch.manual_seed(3)
    t = torch.randn(2, 96, 2, 64).bfloat16()
    r = OA.kmeans_reorder_tokens(t, n_clusters=5, max_iters=4, seed=1)
    bh, s = r.order.shape
    assert (bh, s) == (4, 96)
    ar = torch.arange(s).expand(bh, s)
    assert torch.equal(torch.sort(r.order, dim=1).values, ar)                       # a permutation
    assert torch.equal(torch.gather(r.inverse_order, 1, r.order), ar)               # inverse[order[j]] == j
    sorted_labels = torch.gather(r.labels, 1, r.order)
    assert (sorted_labels[:, 1:] >= sorted_labels[:, :-1]).all()                    # grouped by cluster
    same = sorted_labels[:, 1:] == sorted_labels[:, :-1]
    assert (r.order[:, 1:][same] > r.order[:, :-1][same]).all()                     # stable
    assert r.labels.min() >= 0 and r.labels.max() < 5
    # every token sits with its nearest centroid (Lloyd fixed-point property of the last assignment is
    # not required; the labels must at least be deterministic)
    r2 = OA.kmeans_reorder_tokens(t, n_clusters=5, max_iters=4, seed=1)
    assert torch.equal(r.labels, r2.labels)
    with pytest.raises(ValueError):
        OA.kmeans_reorder_tokens(t, n_clusters=0)


def test_kv_copermutation_preserves_attention():
    """tests/test_v_kmeans.py:39-51 of the reference: cos > 0.9999, max-abs < 1e-2."""
    torch.manual_seed(4)
    q, k, v = (torch.randn(1, 128, 2, 64).bfloat16() for _ in range(3))
    r = OA.kmeans_reorder_tokens(v, n_clusters=4, max_iters=3)
    kp = OA.apply_kv_permutation(k, r.order)
    a = OA.reference_attention(q, k, v).float()
    b = OA.reference_attention(q, kp, r.tensor_reordered).float()
    assert torch.nn.functional.cosine_similarity(a.flatten()[None], b.flatten()[None]).item() > 0.9999
    assert (a - b).abs().max() < 1e-2


@pytest.mark.parametrize("p_quant,rowmax", [("elementwise", "online"), ("dynamic", "online"), ("dynamic", "qm_k"),
                                            ("mx", "online")])
def test_fake_quant_attention_tracks_sdpa(p_quant, rowmax):
    """Floors of the reference's integration sweep (tests/test_fake_quant_attention.py:38-61)."""
    torch.manual_seed(5)
    q, k, v = (torch.randn(1, 256, 2, 64).bfloat16() for _ in range(3))
    cfg = QuantConfig(fp8_block_size=64, q_smooth_block_size=64, q_kmeans_k=4, p_quant=p_quant, rowmax_mode=rowmax,
                      p_mx_block_n=64)
    o = OA.fake_quant_attention(q, k, v, cfg)
    ref = OA.reference_attention(q, k, v)
    assert o.shape == q.shape and o.dtype == q.dtype and torch.isfinite(o.float()).all()
    assert OA.compute_metrics(o, ref)["cosine"] > 0.93


def test_mx_p_is_offset_invariant():
    """tests/test_v_quant_variants.py:111-130 of the reference: exact equality."""
    torch.manual_seed(6)
    q, k, v = (torch.randn(1, 128, 1, 64).bfloat16() for _ in range(3))
    base = dict(fp8_block_size=64, smoothing="off", q_kmeans_k=None, v_quant="mxfp8", p_quant="mx")
    a = OA.fake_quant_attention(q, k, v, QuantConfig(**base, p_max_offset=0), out_fp32=True)
    b = OA.fake_quant_attention(q, k, v, QuantConfig(**base, p_max_offset=8), out_fp32=True)
    assert (a - b).abs().max().item() == 0.0


def test_true_fp8_gap_to_reference_convention_is_small_but_real():
    """fp8_block Q/K: the reference rounds code * scale to BF16 before the MMA, a
    real FP8 MMA does not; mxfp8 scales are powers of two, so there the two agree exactly."""
    torch.manual_seed(7)
    q, k, v = (torch.randn(1, 256, 2, 64).bfloat16() for _ in range(3))
    cfg = QuantConfig(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="elementwise")
    a = OA.fake_quant_attention(q, k, v, cfg, faithful=True, out_fp32=True)
    b = OA.fake_quant_attention(q, k, v, cfg, faithful=False, out_fp32=True)
    m = OA.compute_metrics(b, a)
    assert 0.999 < m["cosine"] and m["max_abs"] > 0
    cfg = QuantConfig(qk_quant="mxfp8", v_quant="mxfp8", smoothing="off", q_kmeans_k=None)
    a = OA.fake_quant_attention(q, k, v, cfg, faithful=True, out_fp32=True)
    b = OA.fake_quant_attention(q, k, v, cfg, faithful=False, out_fp32=True)
    assert (a - b).abs().max().item() == 0.0


def test_errors_match_reference_messages():
    q = torch.randn(1, 64, 1, 64).bfloat16()
    with pytest.raises(ValueError, match="requires cfg.p_requant=True"):
        OA.fake_quant_attention(q, q, q, QuantConfig(p_requant=False, blasst_lambda=0.1))
    with pytest.raises(ValueError, match="requires smoothing='full'"):
        OA.fake_quant_attention(q, q, q, QuantConfig(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None,
                                                     rowmax_mode="qm_k"))
    with pytest.raises(ValueError, match="shapes must match"):
        OA.fake_quant_attention(q, q[:, :32], q, QuantConfig())


def test_rowmax_counters_of_the_oracle():
    """The events bench/count_rowmax_updates_triton.py of the reference counts: every row updates in its first block
    (no rescale: no mass yet), the frozen estimate never updates, the thresholded estimate updates far less often."""
    torch.manual_seed(6)
    q, k, v = (torch.randn(1, 512, 2, 64).bfloat16() for _ in range(3))
    kw = dict(fp8_block_size=64, q_smooth_block_size=64, q_kmeans_k=None, smoothing="full")
    counts = {}
    for name, extra in (("online", dict(p_quant="dynamic")), ("thresholds", dict(p_quant="dynamic", rowmax_mode="qm_k")),
                        ("frozen", dict(rowmax_mode="qm_k"))):
        c = {}
        OA.fake_quant_attention(q, k, v, QuantConfig(**kw, **extra), faithful=False, rowmax_counters=c)
        counts[name] = c
    on, th, fr = counts["online"], counts["thresholds"], counts["frozen"]
    rows = 1 * 512 * 2
    assert on["rows_with_update"] == rows and on["updates"] - on["rescales"] == rows and on["downward_updates"] == 0
    assert 1 <= on["max_updates_per_row"] <= 512 // 64
    assert fr == dict(updates=0, rescales=0, upward_updates=0, downward_updates=0, rows_with_update=0, max_updates_per_row=0)
    assert th["updates"] == th["upward_updates"] + th["downward_updates"] and th["rescales"] * 4 < on["rescales"]


def test_cross_attention_extension_of_the_oracle():
    """K / V of their own length: the oracle's extension (the reference's entry takes equal shapes) tracks plain
    attention over the same keys, and with equal lengths it is the ordinary path."""
    torch.manual_seed(8)
    q = torch.randn(1, 256, 2, 64).bfloat16()
    k = (torch.randn(1, 128, 2, 64) + 1.0).bfloat16()
    v = torch.randn(1, 128, 2, 64).bfloat16()
    cfg = QuantConfig(fp8_block_size=64, q_smooth_block_size=64, q_kmeans_k=None, smoothing="full", p_quant="dynamic",
                      rowmax_mode="qm_k", v_smooth_mode="per_block")
    o = OA.fake_quant_attention(q, k, v, cfg, faithful=False, cross=True)
    assert o.shape == q.shape and torch.isfinite(o.float()).all()
    assert OA.compute_metrics(o, OA.reference_attention(q, k, v))["cosine"] > 0.99
    same = OA.fake_quant_attention(q, q, q, cfg, faithful=False, cross=True)
    assert torch.equal(same, OA.fake_quant_attention(q, q, q, cfg, faithful=False))
    with pytest.raises(ValueError, match="shapes must match"):
        OA.fake_quant_attention(q, k, v, cfg)
    with pytest.raises(ValueError, match="cross-attention wants"):
        OA.fake_quant_attention(q, k, v[:, :64], cfg, cross=True)
