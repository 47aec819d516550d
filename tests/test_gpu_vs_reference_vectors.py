"""The CUDA library against vectors recorded from the reference's OWN Triton kernels on a B200.

``tests/golden/reference_gpu_vectors.pt`` (written by ``tests/golden/make_golden_gpu.py``, which ran the reference
project's kernels on the same GPU architecture) holds, for seeded inputs: the reference quantizers' codes and scales,
its smoothing / rotation outputs, outputs of direct launches of its streaming kernel in every mode, and outputs of
its public entry for whole configurations (k-means labels stored, since its third-party k-means is unavailable).

* Quantizers: codes and scales are compared BYTE FOR BYTE -- this is the "bit-exact against the reference quantizers"
  claim of the project, checked against the reference itself rather than a restatement. The same holds for the
  smoothed tensors, the rotated tensors and the de-quantisers; the FP32 means may differ in the last two ulps (their
  sums run in a different order).
* Streaming kernel, reference operands: ``fake_quant_attention_triton`` is fed the very operands the reference's
  glue built; per element the bound is one BF16 ulp of the reference value (it stores BF16) plus 2e-3 x RMS, the
  cosine must reach 0.99999, and at most ``ATT_FRAC`` of the elements may exceed the bound (a P value on an e4m3
  rounding boundary flips with the last bits of the score). BLASST decisions (the stats tensor) must be identical.
* Whole entry: ``fake_quant_attention(..., _reference_operands=True)`` is held to the same bound; the default
  FP8-code path multiplies the codes themselves, which the reference's BF16 de-quantisation of Q / K cannot
  represent, so its distance is only bounded loosely here and reported.
"""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import ref_gpu_cases as C                                            # noqa: E402
import low_bit_fake_quant as fq                                      # noqa: E402
from low_bit_fake_quant.attention_triton import fake_quant_attention_triton, raise_if_device_error  # noqa: E402
from low_bit_fake_quant.config import QuantConfig                    # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FIXTURE = os.path.join(HERE, "golden", "reference_gpu_vectors.pt")
ATT_FRAC = 2e-3
ATT_FRAC_SDPA = 2e-2


@pytest.fixture(scope="module")
def vec():
    if not os.path.exists(FIXTURE):
        pytest.skip("reference_gpu_vectors.pt has not been recorded")
    return torch.load(FIXTURE, weights_only=False)


def same_bytes(got, want_u8):
    return torch.equal(got.view(torch.uint8).cpu(), want_u8)


def means_close(got, want):
    got, want = got.float().cpu(), want.float()
    tol = 2.0 * torch.finfo(torch.float32).eps * torch.maximum(got.abs(), want.abs()).clamp_min(1e-30)
    return bool(((got - want).abs() <= tol).all())                   # FP32 sums in another order: two ulps


def attention_report(got, want_bf16):
    want = want_bf16.float()
    got = got.float().cpu()
    rms = want.pow(2).mean().sqrt()
    ulp = torch.exp2(torch.floor(torch.log2(want.abs().clamp_min(1e-30)))) * 2.0 ** -7
    over = ((got - want).abs() > ulp + 2e-3 * rms).float().mean().item()
    cos = torch.nn.functional.cosine_similarity(got.flatten()[None], want.flatten()[None]).item()
    return over, cos


@pytest.mark.parametrize("d", [128, 64])
def test_quantizers_are_bit_exact_against_the_reference(vec, d):
    r = vec["quant"][f"d{d}"]
    s, h, _ = r["shape"]
    q, k, v = (t.to(DEV) for t in C.base_inputs(r["seed"], s, h, d))
    for nm, fn, x, kw in (("fp8_block64_q", fq.fp8_block_quant, q, dict(block_s=64)),
                          ("fp8_block128_k", fq.fp8_block_quant, k, dict(block_s=128)),
                          ("fp8_channel_v", fq.fp8_per_channel_quant, v, {}),
                          ("mxfp8_qk_q", fq.mxfp8_qk_quant, q, dict(block_d=32)),
                          ("mxfp8_v_v", fq.mxfp8_v_quant, v, dict(block_s=64)),
                          ("fp8_block64_q_float16", fq.fp8_block_quant, q.to(torch.float16), dict(block_s=64)),
                          ("fp8_block64_q_float32", fq.fp8_block_quant, q.to(torch.float32), dict(block_s=64))):
        c, sc = fn(x, **kw)
        assert torch.equal(sc.cpu(), r[nm]["scale"]), nm
        assert same_bytes(c, r[nm]["codes"]), (nm, (c.view(torch.uint8).cpu() != r[nm]["codes"]).sum().item())
    f8 = lambda u: u.view(torch.float8_e4m3fn).to(DEV)
    assert torch.equal(fq.fp8_block_dequant(f8(r["fp8_block64_q"]["codes"]), r["fp8_block64_q"]["scale"].to(DEV), 64,
                                            dtype=torch.bfloat16).cpu(), r["fp8_block64_q"]["dequant_bf16"])
    assert torch.equal(fq.fp8_per_channel_dequant(f8(r["fp8_channel_v"]["codes"]), r["fp8_channel_v"]["scale"].to(DEV),
                                                  dtype=torch.bfloat16).cpu(), r["fp8_channel_v"]["dequant_bf16"])
    assert torch.equal(fq.mxfp8_qk_dequant(f8(r["mxfp8_qk_q"]["codes"]), r["mxfp8_qk_q"]["scale"].to(DEV), 32,
                                           dtype=torch.bfloat16).cpu(), r["mxfp8_qk_q"]["dequant_bf16"])
    assert torch.equal(fq.mxfp8_v_dequant(f8(r["mxfp8_v_v"]["codes"]), r["mxfp8_v_v"]["scale"].to(DEV), 64,
                                          dtype=torch.bfloat16).cpu(), r["mxfp8_v_v"]["dequant_bf16"])


@pytest.mark.parametrize("d", [128, 64])
def test_smoothing_and_rotation_against_the_reference(vec, d):
    r = vec["quant"][f"d{d}"]
    s, h, _ = r["shape"]
    q, k, v = (t.to(DEV) for t in C.base_inputs(r["seed"], s, h, d))
    ks, mean = fq.smooth_k(k)
    assert torch.equal(ks.cpu(), r["smooth_k"]["out"]) and means_close(mean, r["smooth_k"]["mean"])
    qs, qm = fq.group_mean_q(q, block_q=128)
    assert torch.equal(qs.cpu(), r["group_mean_q128"]["out"]) and means_close(qm, r["group_mean_q128"]["qm"])
    vs, va = fq.smooth_v_per_block(v, block_s=64)
    assert torch.equal(vs.cpu(), r["smooth_v64"]["out"]) and means_close(va, r["smooth_v64"]["alpha"])
    qh, kh = fq.apply_qk_hadamard(q, k, random_sign=True, seed=0)
    assert torch.equal(qh.cpu(), r["hadamard"]["q"]) and torch.equal(kh.cpu(), r["hadamard"]["k"])


def _k12_case_names():
    return [f"d128/{n}" for n in C.K12_CASES] + [f"d64/{n}" for n in C.K12_CASES_D64]


@pytest.mark.parametrize("name", _k12_case_names())
def test_direct_launch_against_the_reference_kernel(vec, name):
    rec = vec["k12"][name]
    if "error" in rec:
        pytest.skip(f"the reference's own kernel failed for this case when the vectors were recorded: {rec['error'][:80]}")
    pool = vec["pool"]
    ops = [pool[k].to(DEV) for k in rec["ops"]]
    kw = {a: (pool[b].to(DEV) if tag == "T" else b) for a, (tag, b) in rec["kw"].items()}
    got = fake_quant_attention_triton(*ops, **kw)
    raise_if_device_error(torch.device(DEV))
    if kw.get("return_blasst_stats", False):
        got, stats = got
        assert torch.equal(stats.cpu(), rec["stats"]), name
    over, cos = attention_report(got, rec["out"])
    assert cos >= 0.99999 and over <= ATT_FRAC, (name, cos, over)


@pytest.mark.parametrize("name", list(C.ENTRY_CASES))
def test_whole_entry_against_the_reference(vec, name):
    s, h, d = C.ENTRY_SHAPE
    q, k, v = (t.to(DEV) for t in C.base_inputs(300, s, h, d))
    lab = vec["entry"]["labels"]
    cfg = QuantConfig(**C.ENTRY_CASES[name])
    kw = {}
    if cfg.q_kmeans_k is not None:
        kw["_q_labels"] = lab["q"].to(torch.int32).to(DEV)
    if cfg.v_kmeans_k is not None:
        kw["_v_labels"] = lab["v"].to(torch.int32).to(DEV)
    want = vec["entry"][name]["out"]
    got = fq.fake_quant_attention(q, k, v, cfg, _reference_operands=True, **kw)
    raise_if_device_error(torch.device(DEV))
    over, cos = attention_report(got, want)
    assert cos >= 0.99999 and over <= (ATT_FRAC if cfg.p_requant else ATT_FRAC_SDPA), (name, cos, over)
    if cfg.p_requant:
        # the default path: the e4m3 codes themselves are multiplied (exact scales outside the MMA)
        fp8 = fq.fake_quant_attention(q, k, v, cfg, **kw)
        raise_if_device_error(torch.device(DEV))
        _, cos8 = attention_report(fp8, want)
        assert cos8 >= 0.9995, (name, cos8)
