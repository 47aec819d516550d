"""GPU parity of the quantizer / preprocess kernels against the CPU oracle.

Codes and scales must be BIT-EXACT on identical inputs. The library follows the arithmetic of the reference's
kernels on the GPU (``x * rcp.approx(scale)``; it is bit-identical to codes recorded from them, see
``test_gpu_vs_reference_vectors.py``); the oracle does the same here because ``conftest.py`` hands it the GPU's
reciprocal (``oracle.quant_ops.set_reciprocal``) -- on a machine without a GPU it divides by IEEE rules, which rounds
to a neighbouring code in about one element per million. Means are FP32 sums whose order differs from the oracle's,
so they get an ulp bound and the centred tensors a mismatch-count bound.
"""
import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant import _lib as L
from low_bit_fake_quant.attention_triton import qm_corr
from low_bit_fake_quant.kmeans import kmeans_labels
from oracle import api as OA
from oracle import quant_ops as OQ

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(B, S, H, D, dtype, seed=0):
    torch.manual_seed(seed)
    x = torch.randn(B, S, H, D)
    x[..., :4] *= 10.0                       # outlier channels
    x = x + 0.5 * torch.randn(1, 1, H, D)
    x[0, 0, 0, :8] = 0.0
    return x.to(dtype)


def _same_codes(got, want, max_frac=0.0):
    """Equal codes; with ``max_frac`` > 0, at most that fraction may differ, each by one code step (same sign)."""
    g, w = got.view(torch.uint8).cpu().to(torch.int16), want.view(torch.uint8).to(torch.int16)
    diff = g != w
    if not diff.any():
        return True
    if max_frac <= 0.0 or diff.float().mean().item() > max_frac:
        return False
    return bool(((g[diff] - w[diff]).abs() == 1).all())


FP32_SCALE_CODES = 0.0           # see the module docstring: exact, as long as the oracle has the GPU's reciprocal


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("D,blk", [(128, 64), (64, 128), (128, 32)])
def test_fp8_block_bit_exact(dtype, D, blk):
    x = _inputs(2, 256, 3, D, dtype)
    c, s = fq.fp8_block_quant(x.to(DEV), blk)
    oc, os_ = OQ.fp8_block_quant(x, blk)
    assert _same_codes(c, oc, FP32_SCALE_CODES) and torch.equal(s.cpu(), os_)
    for out_dt in (torch.bfloat16, torch.float32):
        assert torch.equal(fq.fp8_block_dequant(c, s, blk, dtype=out_dt).cpu(), OQ.fp8_block_dequant(c.cpu(), os_, blk, dtype=out_dt))


def test_fp8_block_layouts_and_padding():
    x = _inputs(1, 192, 2, 128, torch.bfloat16, seed=1)
    oc, _ = OQ.fp8_block_quant(x, 64)
    c, _ = fq.fp8_block_quant(x.to(DEV), 64, _layout=L.LAYOUT_BHSD, _s_pad=256)
    assert _same_codes(c[:, :, :192].permute(0, 2, 1, 3).contiguous(), oc, FP32_SCALE_CODES)
    assert int(c.view(torch.uint8)[:, :, 192:].sum()) == 0
    c, _ = fq.fp8_block_quant(x.to(DEV), 64, _layout=L.LAYOUT_BHDS, _s_pad=256)
    assert _same_codes(c[..., :192].permute(0, 3, 1, 2).contiguous(), oc, FP32_SCALE_CODES)
    assert int(c.view(torch.uint8)[..., 192:].sum()) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fp8_channel_bit_exact(dtype):
    x = _inputs(2, 320, 2, 128, dtype, seed=2)        # S not a multiple of the kernel's row tiles
    c, s = fq.fp8_per_channel_quant(x.to(DEV))
    oc, os_ = OQ.fp8_per_channel_quant(x)
    assert _same_codes(c, oc, FP32_SCALE_CODES) and torch.equal(s.cpu(), os_)
    assert torch.equal(fq.fp8_per_channel_dequant(c, s, dtype=torch.bfloat16).cpu(), OQ.fp8_per_channel_dequant(c.cpu(), os_, dtype=torch.bfloat16))
    ct, _ = fq.fp8_per_channel_quant(x.to(DEV), _layout=L.LAYOUT_BHDS, _s_pad=384)
    assert _same_codes(ct[..., :320].permute(0, 3, 1, 2).contiguous(), c.cpu())


@pytest.mark.parametrize("D,blk", [(128, 32), (64, 32), (128, 64), (128, 16)])
def test_mxfp8_qk_bit_exact(D, blk):
    x = _inputs(1, 200, 3, D, torch.bfloat16, seed=3)
    c, s = fq.mxfp8_qk_quant(x.to(DEV), blk)
    oc, os_ = OQ.mxfp8_qk_quant(x, blk)
    assert _same_codes(c, oc) and torch.equal(s.cpu(), os_)
    assert torch.equal(fq.mxfp8_qk_dequant(c, s, blk, dtype=torch.bfloat16).cpu(), OQ.mxfp8_qk_dequant(oc, os_, blk, dtype=torch.bfloat16))


def test_mxfp8_pow2_edge_cases():
    # block amax exactly 448 * 2^k (scale 2^k) and one BF16 step above it (scale 2^(k+1))
    x = torch.zeros(1, 4, 1, 128)
    x[0, 0, 0, 0] = 448.0
    x[0, 1, 0, 0] = 450.0
    x[0, 2, 0, 32] = 3.5
    x[0, 3, 0, 64] = 1.75 * 2 ** -6
    x = x.bfloat16()
    c, s = fq.mxfp8_qk_quant(x.to(DEV), 32)
    oc, os_ = OQ.mxfp8_qk_quant(x, 32)
    assert _same_codes(c, oc) and torch.equal(s.cpu(), os_)
    assert s[0, 0, 0, 0].item() == 1.0 and s[0, 1, 0, 0].item() == 2.0


@pytest.mark.parametrize("blk", [32, 64])
def test_mxfp8_v_bit_exact(blk):
    x = _inputs(2, 256, 2, 128, torch.bfloat16, seed=4)
    c, s = fq.mxfp8_v_quant(x.to(DEV), blk)
    oc, os_ = OQ.mxfp8_v_quant(x, blk)
    assert _same_codes(c, oc) and torch.equal(s.cpu(), os_)
    assert torch.equal(fq.mxfp8_v_dequant(c, s, blk, dtype=torch.bfloat16).cpu(), OQ.mxfp8_v_dequant(oc, os_, blk, dtype=torch.bfloat16))
    ct, _ = fq.mxfp8_v_quant(x.to(DEV), blk, _layout=L.LAYOUT_BHDS, _s_pad=256)
    assert _same_codes(ct.permute(0, 3, 1, 2).contiguous(), oc)


def test_quantizer_errors():
    x = torch.zeros(1, 100, 1, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="divisible"):
        fq.fp8_block_quant(x, 64)
    with pytest.raises(ValueError, match="64 or 128"):
        fq.fp8_block_quant(torch.zeros(1, 64, 1, 96, dtype=torch.bfloat16, device=DEV), 64)
    with pytest.raises(TypeError):
        fq.fp8_block_dequant(x, torch.zeros(1, 1, 1, device=DEV), 100)


def _close_tensor(got, want, max_frac):
    diff = (got.float().cpu() != want.float())
    return diff.float().mean().item() <= max_frac


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_smoothing_kernels(dtype):
    x = _inputs(2, 512, 2, 128, dtype, seed=5)
    o, m = fq.smooth_k(x.to(DEV))
    oo, om = OQ.smooth_k(x)
    assert o.dtype == dtype and m.shape == (2, 2, 128)
    torch.testing.assert_close(m.cpu(), om, rtol=0, atol=2e-6)
    assert _close_tensor(o, oo, 1e-3)                 # a 1-ulp mean difference may flip a BF16 rounding
    assert (o.float().cpu() - oo.float()).abs().max() <= 0.0625
    for blk, fn, ofn in ((256, fq.group_mean_q, OQ.group_mean_q), (64, fq.smooth_v_per_block, OQ.smooth_v_per_block)):
        o, m = fn(x.to(DEV), blk)
        oo, om = ofn(x, blk)
        assert m.shape == (2, 512 // blk, 2, 128)
        torch.testing.assert_close(m.cpu(), om, rtol=0, atol=2e-6)
        assert _close_tensor(o, oo, 1e-3)
    with pytest.raises(ValueError, match="divisible"):
        fq.group_mean_q(x.to(DEV), 100)


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.float16), (128, torch.float32)])
def test_hadamard_bit_exact(D, dtype):
    q = _inputs(2, 64, 3, D, dtype, seed=6)
    k = _inputs(2, 64, 3, D, dtype, seed=7)
    for rs in (True, False):
        gq, gk = fq.apply_qk_hadamard(q.to(DEV), k.to(DEV), random_sign=rs, seed=5)
        oq, ok = OQ.apply_qk_hadamard(q, k, random_sign=rs, seed=5)
        assert torch.equal(gq.cpu(), oq) and torch.equal(gk.cpu(), ok)
    # sharded rotation uses the global head's signs
    gq, _ = fq.apply_qk_hadamard(q[:, :, 1:].contiguous().to(DEV), k[:, :, 1:].contiguous().to(DEV), seed=5, head_offset=1, total_heads=3)
    oq, _ = OQ.apply_qk_hadamard(q, k, seed=5)
    assert torch.equal(gq.cpu(), oq[:, :, 1:])


def test_reorder_bit_exact_given_labels():
    x = _inputs(2, 300, 2, 128, torch.bfloat16, seed=8)
    labels = torch.randint(0, 7, (4, 300))
    r = fq.kmeans_reorder_tokens(x.to(DEV), n_clusters=7, labels=labels.to(DEV).int())
    o = OA.reorder_from_labels(x, labels)
    assert torch.equal(r.order.cpu(), o.order) and torch.equal(r.inverse_order.cpu(), o.inverse_order)
    assert torch.equal(r.tensor_reordered.cpu(), o.tensor_reordered)
    assert r.order.dtype == torch.int64 and r.labels.dtype == torch.int64
    kp = fq.apply_kv_permutation(x.to(DEV), r.order)
    assert torch.equal(kp.cpu(), OA.apply_kv_permutation(x, o.order))


def test_kmeans_labels_invariants_and_oracle_agreement():
    torch.manual_seed(9)
    centers = 4.0 * torch.randn(6, 128)
    x = (centers[torch.randint(0, 6, (2, 512, 2))] + 0.3 * torch.randn(2, 512, 2, 128)).bfloat16()
    g1 = kmeans_labels(x.to(DEV), n_clusters=6, max_iters=6, seed=3)
    g2 = kmeans_labels(x.to(DEV), n_clusters=6, max_iters=6, seed=3)
    assert torch.equal(g1, g2)                                         # bit-reproducible
    assert g1.shape == (4, 512) and int(g1.min()) >= 0 and int(g1.max()) < 6
    want = OA.lloyd_labels(x.permute(0, 2, 1, 3).reshape(4, 512, 128).float(), 6, 6, 3)
    assert (g1.cpu().long() == want).float().mean().item() > 0.99
    # sharding: head 1 alone, told where it sits, reproduces head 1 of the full run
    g3 = kmeans_labels(x[:, :, 1:].contiguous().to(DEV), n_clusters=6, max_iters=6, seed=3, head_offset=1, total_heads=2)
    assert torch.equal(g3, g1[1::2])


@pytest.mark.parametrize("k,D", [(32, 128), (64, 128), (5, 64)])
def test_kmeans_tensor_core_assignment_agrees_with_fp32_assignment(k, D, monkeypatch):
    """BF16 tokens take the tensor-core assignment (centroids split into three BF16 pieces); the FP32 FFMA
    assignment is the cross-check. They differ only in summation order, i.e. on near-ties."""
    torch.manual_seed(k + D)
    x = (torch.randn(2, 1000, 3, D) + 2.0 * torch.randn(1, 1, 3, D)).bfloat16().to(DEV)      # ragged last tile
    L.set_flag(L.FLAG_KMEANS_FFMA, False)
    tc = kmeans_labels(x, n_clusters=k, max_iters=5, seed=1)
    assert torch.equal(tc, kmeans_labels(x, n_clusters=k, max_iters=5, seed=1))               # reproducible
    L.set_flag(L.FLAG_KMEANS_FFMA, True)
    ff = kmeans_labels(x, n_clusters=k, max_iters=5, seed=1)
    assert int(tc.min()) >= 0 and int(tc.max()) < k
    assert (tc == ff).float().mean().item() > 0.995
    # D = 128: the centroid sums are taken inside the assignment kernel (one-hot x tokens on the tensor cores); the
    # update by sort + segment means is the cross-check. Same sums up to summation order.
    L.set_flag(L.FLAG_KMEANS_FFMA, False)
    L.set_flag(L.FLAG_KMEANS_SORTED, True)
    srt = kmeans_labels(x, n_clusters=k, max_iters=5, seed=1)
    assert (tc == srt).float().mean().item() > 0.995


def test_qm_corr_and_rowmax():
    torch.manual_seed(10)
    qm = torch.randn(2, 3, 2, 128)
    ks = _inputs(2, 200, 2, 128, torch.bfloat16, seed=11)
    corr, rm = qm_corr(qm.to(DEV), ks.to(DEV), sm_scale=0.0884, s_pad=256, want_rowmax=True)
    ref = torch.einsum("bghd,bshd->bhgs", qm, ks.float()) * 0.0884
    torch.testing.assert_close(corr[..., :200].cpu(), ref, rtol=1e-5, atol=1e-4)
    assert float(corr[..., 200:].abs().sum()) == 0.0
    torch.testing.assert_close(rm.cpu(), ref.amax(-1), rtol=1e-5, atol=1e-4)
    est = OA.estimate_rowmax_from_qm_k(qm, ks, block_q=64, sm_scale=0.0884)      # (B,H,G*64) needs S == G*64
    assert est.shape[-1] == 192


@pytest.mark.parametrize("S,G,D", [(200, 3, 128), (2304, 9, 128), (4096, 130, 64), (1000, 5, 64)])
def test_qm_corr_tensor_core_kernel_agrees_with_fp32_kernel(S, G, D, monkeypatch):
    """BF16 keys take the tensor-core kernel (group means split into three BF16 pieces: exact products, FP32 sums);
    the FP32 FFMA kernel is the cross-check. More than 128 groups span two CTAs along the group axis; a ragged last
    key tile and the zero-filled columns up to ``s_pad`` are covered."""
    torch.manual_seed(S + G)
    qm = torch.randn(2, G, 3, D, device=DEV)
    ks = (torch.randn(2, S, 3, D, device=DEV) * 2).bfloat16()
    s_pad = (S + 63) // 64 * 64
    L.set_flag(L.FLAG_QM_CORR_FFMA, False)
    c_tc, r_tc = qm_corr(qm, ks, sm_scale=0.0884, s_pad=s_pad, want_rowmax=True)
    c_tc2, _ = qm_corr(qm, ks, sm_scale=0.0884, s_pad=s_pad)
    assert torch.equal(c_tc, c_tc2)                                            # reproducible
    L.set_flag(L.FLAG_QM_CORR_FFMA, True)
    c_ff, r_ff = qm_corr(qm, ks, sm_scale=0.0884, s_pad=s_pad, want_rowmax=True)
    ref = torch.einsum("bghd,bshd->bhgs", qm.double(), ks.double()) * 0.0884
    assert float(c_tc[..., S:].abs().sum()) == 0.0
    err_tc = (c_tc[..., :S].double() - ref).abs().max().item()
    err_ff = (c_ff[..., :S].double() - ref).abs().max().item()
    assert err_tc <= max(2.0 * err_ff, 1e-5), (err_tc, err_ff)                  # as accurate as the FP32 kernel
    torch.testing.assert_close(c_tc, c_ff, rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(r_tc, c_tc[..., :S].amax(-1), rtol=0, atol=0)   # the row max is the max of what was stored
    torch.testing.assert_close(r_tc, r_ff, rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("S,D,k", [(96, 64, 4), (130, 128, 5), (1025, 128, 64)])
def test_kmeans_short_and_ragged_slabs(S, D, k):
    """A slab shorter than one 128-token tile, one token past a tile, one token past a CTA's eight tiles: the
    tensor-core assignment, the chunked sort and the two-step means against the oracle's Lloyd loop."""
    torch.manual_seed(S)
    x = torch.randn(2, S, 3, D).bfloat16()
    got = kmeans_labels(x.to(DEV), n_clusters=k, max_iters=4, seed=1)
    want = OA.lloyd_labels(x.permute(0, 2, 1, 3).reshape(6, S, D).float(), k, 4, 1)
    assert int(got.min()) >= 0 and int(got.max()) < k
    assert (got.cpu().long() == want).float().mean().item() > 0.99


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_quantizers_keep_the_sign_of_zero_and_small_values(dtype):
    """FP16 inputs underflow to +-0; -0 / scale is -0 (code 0x80), which the reciprocal-and-correction division has to
    hand to the plain division to get right. Codes are compared as bytes."""
    torch.manual_seed(5)
    x = (torch.randn(2, 128, 2, 128) * 1e-4)
    x[:, ::3] = -0.0
    x[:, 1::7] *= 1e-5                                   # below the FP16 range: +-0 after the cast
    x = x.to(dtype)
    c, s = fq.fp8_block_quant(x.to(DEV), 64)
    oc, os_ = OQ.fp8_block_quant(x, 64)
    assert torch.equal(c.cpu().view(torch.uint8), oc.view(torch.uint8)) and torch.equal(s.cpu(), os_)
    c, s = fq.fp8_per_channel_quant(x.to(DEV))
    oc, os_ = OQ.fp8_per_channel_quant(x)
    assert torch.equal(c.cpu().view(torch.uint8), oc.view(torch.uint8)) and torch.equal(s.cpu(), os_)
    assert int((oc.view(torch.uint8) == 0x80).sum()) > 0          # the case does hold negative zeros
