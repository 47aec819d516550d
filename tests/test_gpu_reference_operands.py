"""The reference's own operand convention on the GPU: Q / K de-quantised to BF16, V as BF16 code values, Q.K^T and
P.V as BF16 MMAs (`fake_quant_attention_triton`, the reference's direct-launch signature, and
`fake_quant_attention(..., _reference_operands=True)` which builds those operands the way attention.py:505-639
does). Checked against the oracle in the same convention (`faithful=True`), to the tolerance of the task."""
import zlib

import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant.attention_triton import fake_quant_attention_triton, raise_if_device_error
from low_bit_fake_quant.config import QuantConfig
from oracle import api as OA

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
COMMON = dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, q_smooth_block_size=256)

CASES = {
    "k_only_static_online": dict(smoothing="k_only", q_kmeans_k=None),
    "dynamic_online": dict(smoothing="k_only", q_kmeans_k=None, p_quant="dynamic"),
    "mx_p": dict(smoothing="k_only", q_kmeans_k=None, p_quant="mx", p_mx_block_n=64),
    "full_smoothing": dict(smoothing="full", q_kmeans_k=None),
    "v_alpha": dict(smoothing="k_only", q_kmeans_k=None, v_smooth_mode="per_block"),
    "full_stack_dynamic_qm_k": dict(smoothing="full", q_kmeans_k=8, v_kmeans_k=8, v_smooth_mode="per_block",
                                    p_quant="dynamic", rowmax_mode="qm_k"),
    "qm_k_frozen_estimate": dict(smoothing="full", q_kmeans_k=None, rowmax_mode="qm_k"),
    "mxfp8_all_hadamard": dict(qk_quant="mxfp8", v_quant="mxfp8", smoothing="off", q_kmeans_k=None, qk_hadamard=True),
    "bn32": dict(smoothing="k_only", q_kmeans_k=None, p_requant_block_m=32, p_requant_block_n=32, p_quant="dynamic"),
}


def _qkv(B, S, H, D, seed):
    torch.manual_seed(seed)
    q, k, v = torch.randn(B, S, H, D), torch.randn(B, S, H, D), torch.randn(B, S, H, D)
    k = k + 2.0 * torch.randn(1, 1, H, D)
    return q.bfloat16(), k.bfloat16(), v.bfloat16()


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("D,S", [(128, 512), (64, 1280)])
def test_reference_operand_mode_matches_the_oracle_in_the_reference_convention(name, D, S):
    cfg = QuantConfig(**{**COMMON, **CASES[name]})
    q, k, v = _qkv(1, S, 2, D, seed=zlib.crc32(name.encode()) % 1000)
    g = fq.fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg, _debug_fp32=True, _reference_operands=True)
    raise_if_device_error(torch.device(DEV))
    ql = vl = None
    if cfg.q_kmeans_k is not None or cfg.v_kmeans_k is not None:
        pc = fq.prepare_for_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg)
        ql = pc.q_kmeans.labels.cpu() if pc.q_kmeans is not None else None
        vl = pc.v_kmeans.labels.cpu() if pc.v_kmeans is not None else None
    o = OA.fake_quant_attention(q, k, v, cfg, faithful=True, out_fp32=True, q_labels=ql, v_labels=vl)
    g = g.float().cpu()
    assert torch.isfinite(g).all()
    rep = OA.parity_report(g, o, q, k, v)
    assert OA.parity_ok(rep), rep


def test_reference_operand_mode_closes_the_gap_to_the_reference_convention():
    """Element-wise, the FP8-code kernel sits at cosine ~0.9999 from the reference's convention (the BF16 rounding
    of the de-quantised Q / K); the BF16-operand mode is an order of magnitude closer in max-abs error."""
    q, k, v = _qkv(1, 1024, 2, 128, seed=13)
    cfg = QuantConfig(**COMMON, smoothing="k_only", q_kmeans_k=None)
    o = OA.fake_quant_attention(q, k, v, cfg, faithful=True, out_fp32=True)
    codes = fq.fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg, _debug_fp32=True).float().cpu()
    ref_ops = fq.fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg, _debug_fp32=True, _reference_operands=True).float().cpu()
    m_codes, m_ref = OA.compute_metrics(codes, o), OA.compute_metrics(ref_ops, o)
    assert m_ref["cosine"] >= 0.99999 and m_ref["rmse"] < 0.2 * m_codes["rmse"]


def test_direct_launch_signature_and_errors():
    B, H, S, D = 1, 2, 256, 64
    torch.manual_seed(3)
    q, k, v = (torch.randn(B, H, S, D, device=DEV).bfloat16() for _ in range(3))
    ones = torch.ones(B, H, D, device=DEV)
    out = fake_quant_attention_triton(q, k, v, ones, sm_scale=D ** -0.5, p_max_offset=8)
    assert out.shape == (B, H, S, D) and out.dtype == torch.bfloat16 and torch.isfinite(out.float()).all()
    # a per-block V scale wants V as e4m3 code values (random BF16 values are not)
    with pytest.raises(ValueError, match="e4m3 code values"):
        fake_quant_attention_triton(q, k, v, ones, sm_scale=1.0, p_max_offset=8,
                                    v_block_scale_bsh=torch.ones(B, S // 64, H, device=DEV), v_block_size=64)
    with pytest.raises(ValueError, match="multiple of block_n"):
        fake_quant_attention_triton(q, k, v, ones, sm_scale=1.0, p_max_offset=8,
                                    v_block_scale_bsh=torch.ones(B, S // 32, H, device=DEV), v_block_size=32)
    # BLASST and the stats tensor through the direct-launch signature: V as code values
    vc = v.to(torch.float8_e4m3fn).to(torch.bfloat16)
    out, stats = fake_quant_attention_triton(q, k, vc, ones, sm_scale=D ** -0.5, p_max_offset=8, blasst_lambda=0.1,
                                             blasst_fill_mode="mean_a1.5", return_blasst_stats=True)
    assert out.shape == (B, H, S, D) and stats.shape == (S // 64, B * H, 2) and float(stats[..., 1].sum()) == B * H * S * (S // 64)
    with pytest.raises(ValueError, match="blasst_lambda must be in"):
        fake_quant_attention_triton(q, k, vc, ones, sm_scale=1.0, p_max_offset=8, blasst_lambda=1.5)
    with pytest.raises(ValueError, match="requires blasst_lambda"):
        fake_quant_attention_triton(q, k, vc, ones, sm_scale=1.0, p_max_offset=8, blasst_fill_mode="mean")
    with pytest.raises(ValueError, match="v_smooth_block must be > 0"):
        fake_quant_attention_triton(q, k, v, ones, sm_scale=1.0, p_max_offset=8, v_alpha=torch.zeros(B, S // 64, H, D, device=DEV))
    with pytest.raises(ValueError, match="k_smooth_bhsd required"):
        fake_quant_attention_triton(q, k, v, ones, sm_scale=1.0, p_max_offset=8, qm_bhgd=torch.zeros(B, H, 1, D, device=DEV), q_smooth_block=256)
    with pytest.raises(TypeError):
        fake_quant_attention_triton(q.float(), k, v, ones, sm_scale=1.0, p_max_offset=8)
