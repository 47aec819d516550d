"""`prepare_qkv` (src/low_bit_fake_quant/pipeline.py:42-110 of the reference): the public surface on which the
quantizers' codes and scales are observable. Codes and scales must be bit-exact against the oracle's composition of
the same steps; the Q.K-mean correction is an FP32 product cast to `correction_dtype`."""
import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant.config import QuantConfig
from oracle import api as OA
from oracle import quant_ops as Q

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = {
    "fp8_block_channel_k_only": dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, smoothing="k_only",
                                     q_kmeans_k=None),
    "fp8_block_full_kmeans": dict(qk_quant="fp8_block", v_quant="fp8_block", fp8_block_size=128, v_fp8_block_size=64,
                                  smoothing="full", q_smooth_block_size=128, q_kmeans_k=6),
    "mxfp8_hadamard_off": dict(qk_quant="mxfp8", v_quant="mxfp8", smoothing="off", q_kmeans_k=None, qk_hadamard=True),
}


def _bits(t):
    return t.contiguous().view(torch.uint8).cpu()


@pytest.mark.parametrize("name", sorted(CASES))
def test_prepare_qkv_codes_and_scales_are_bit_exact(name):
    cfg = QuantConfig(**CASES[name])
    torch.manual_seed(5)
    q, k, v = (torch.randn(2, 512, 3, 128).bfloat16() for _ in range(3))
    k = (k.float() + 1.5 * torch.randn(1, 1, 3, 128)).bfloat16()
    got = fq.prepare_qkv(q.to(DEV), k.to(DEV), v.to(DEV), cfg)

    qw, kw, vw = q, k, v
    if cfg.q_kmeans_k is not None:
        assert got.kmeans is not None
        km = OA.kmeans_reorder_tokens(q, n_clusters=cfg.q_kmeans_k, labels=got.kmeans.labels.cpu())
        assert torch.equal(got.kmeans.order.cpu(), km.order)
        qw = km.tensor_reordered
    want_qm = want_kmean = None
    if cfg.smoothing in ("k_only", "full"):
        kw, want_kmean = Q.smooth_k(kw)
    if cfg.smoothing == "full":
        qw, want_qm = Q.group_mean_q(qw, block_q=cfg.q_smooth_block_size)
        want_corr = torch.einsum("bqhd,bshd->bqhs", want_qm.float(), kw.float()).to(cfg.correction_dtype)
        assert got.correction.dtype == cfg.correction_dtype and got.correction.shape == want_corr.shape
        assert torch.allclose(got.correction.float().cpu(), want_corr.float(), rtol=2e-3, atol=2e-3)
        assert torch.allclose(got.qm.cpu(), want_qm, rtol=0, atol=1e-6)
    else:
        assert got.qm is None and got.correction is None
    if want_kmean is not None:
        assert torch.allclose(got.k_mean.cpu().float(), want_kmean.float(), rtol=0, atol=1e-6)
    if cfg.qk_hadamard:
        qw, kw = Q.apply_qk_hadamard(qw, kw, random_sign=cfg.qk_hadamard_random_sign, seed=cfg.qk_hadamard_seed)
    qc, qs, _ = OA.quant_qk(qw, cfg)
    kc, ks, _ = OA.quant_qk(kw, cfg)
    vc, vs, _ = OA.quant_v(vw, cfg)
    for g, w in ((got.q, qc), (got.k, kc), (got.v, vc)):
        assert g.dtype == torch.float8_e4m3fn and torch.equal(_bits(g), _bits(w))
    for g, w in ((got.q_scale, qs), (got.k_scale, ks), (got.v_scale, vs)):
        assert g.shape == w.shape and torch.equal(g.cpu(), w)


def test_prepare_qkv_errors():
    x = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="shapes must match"):
        fq.prepare_qkv(x, x[:, :64], x, QuantConfig())
    with pytest.raises(ValueError, match="unsupported qk_quant"):
        fq.prepare_qkv(x, x, x, QuantConfig(qk_quant="int4", smoothing="off", q_kmeans_k=None))
    with pytest.raises(ValueError, match="must live on CUDA"):
        fq.prepare_qkv(x.cpu(), x.cpu(), x.cpu(), QuantConfig())
