"""The CPU oracle against vectors recorded from the reference's OWN Triton kernels on a B200.

``tests/golden/reference_gpu_vectors.pt`` was written by ``tests/golden/make_golden_gpu.py`` (which imports the
reference project and runs its quantizers, smoothing kernels, Hadamard rotation, streaming kernel and public entry
on a GPU). These tests pin ``oracle/quant_ops.py``, ``oracle/k12.py`` and ``oracle/api.py`` to it, on CPU.

Tolerances, and why:
* scales, power-of-two-scaled codes, smoothed tensors, rotated tensors, de-quantised tensors: bit-exact;
* FP32-scaled codes: the GPU divides with an approximate reciprocal no CPU can restate; the IEEE quotient rounds to a
  neighbouring e4m3 code in a few elements per million (``CODE_FRAC``);
* means: FP32 sums in a different order, one ulp;
* attention outputs: the reference stores BF16, so the bound per element is one BF16 ulp of the reference value plus
  the path's stated tolerance 2e-3 x RMS, the cosine must reach 0.99999, and a small fraction of elements (rows in
  which one P value sat on an e4m3 rounding boundary: ``exp2`` of a CPU and ``ex2.approx`` of a GPU differ in the
  last bits) may exceed the bound (``ATT_FRAC``). The ``p_requant=False`` configurations end in torch's SDPA, whose
  GPU kernel (flash attention) and CPU path round P and the partial sums to BF16 at different points: they get
  ``ATT_FRAC_SDPA``.
"""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import ref_gpu_cases as C                         # noqa: E402
from low_bit_fake_quant.config import QuantConfig  # noqa: E402
from oracle import api as OA                       # noqa: E402
from oracle import quant_ops as OQ                 # noqa: E402
from oracle.k12 import k12_attention               # noqa: E402

FIXTURE = os.path.join(HERE, "golden", "reference_gpu_vectors.pt")
CODE_FRAC = 2e-5
ATT_FRAC = 2e-3
ATT_FRAC_SDPA = 2e-2


@pytest.fixture(scope="module")
def vec():
    if not os.path.exists(FIXTURE):
        pytest.skip("reference_gpu_vectors.pt has not been recorded")
    return torch.load(FIXTURE, weights_only=False)


def codes_close(got, want_u8, max_frac):
    g = got.view(torch.uint8).to(torch.int16)
    w = want_u8.to(torch.int16)
    bad = g != w
    if not bad.any():
        return True
    return bad.float().mean().item() <= max_frac and bool(((g - w)[bad].abs() == 1).all())


def ulp_close(a, b, ulps=1):
    a, b = a.float(), b.float()
    tol = ulps * torch.finfo(torch.float32).eps * torch.maximum(a.abs(), b.abs()).clamp_min(1e-30)
    return bool(((a - b).abs() <= tol).all())


def attention_report(got_fp32, want_bf16):
    """Fraction of elements beyond (1 BF16 ulp of the reference + 2e-3 RMS), and the cosine."""
    want = want_bf16.float()
    got = got_fp32.float()
    rms = want.pow(2).mean().sqrt()
    ulp = torch.exp2(torch.floor(torch.log2(want.abs().clamp_min(1e-30)))) * 2.0 ** -7
    over = ((got - want).abs() > ulp + 2e-3 * rms).float().mean().item()
    cos = torch.nn.functional.cosine_similarity(got.flatten()[None], want.flatten()[None]).item()
    return over, cos


@pytest.mark.parametrize("d", [128, 64])
def test_quantizers_and_preprocessing(vec, d):
    r = vec["quant"][f"d{d}"]
    s, h, _ = r["shape"]
    q, k, v = C.base_inputs(r["seed"], s, h, d)
    for nm, fn, x, kw, exact in (("fp8_block64_q", OQ.fp8_block_quant, q, dict(block_s=64), False),
                                 ("fp8_block128_k", OQ.fp8_block_quant, k, dict(block_s=128), False),
                                 ("fp8_channel_v", OQ.fp8_per_channel_quant, v, {}, False),
                                 ("mxfp8_qk_q", OQ.mxfp8_qk_quant, q, dict(block_d=32), True),
                                 ("mxfp8_v_v", OQ.mxfp8_v_quant, v, dict(block_s=64), True),
                                 ("fp8_block64_q_float16", OQ.fp8_block_quant, q.to(torch.float16), dict(block_s=64), False),
                                 ("fp8_block64_q_float32", OQ.fp8_block_quant, q.to(torch.float32), dict(block_s=64), False)):
        c, sc = fn(x, **kw)
        assert torch.equal(sc, r[nm]["scale"]), nm                          # scales: bit-exact
        assert codes_close(c, r[nm]["codes"], 0.0 if exact else CODE_FRAC), nm
    # de-quantisers on the recorded codes and scales: bit-exact
    f8 = lambda u: u.view(torch.float8_e4m3fn)
    assert torch.equal(OQ.fp8_block_dequant(f8(r["fp8_block64_q"]["codes"]), r["fp8_block64_q"]["scale"], 64, dtype=torch.bfloat16),
                       r["fp8_block64_q"]["dequant_bf16"])
    assert torch.equal(OQ.fp8_per_channel_dequant(f8(r["fp8_channel_v"]["codes"]), r["fp8_channel_v"]["scale"], dtype=torch.bfloat16),
                       r["fp8_channel_v"]["dequant_bf16"])
    assert torch.equal(OQ.mxfp8_qk_dequant(f8(r["mxfp8_qk_q"]["codes"]), r["mxfp8_qk_q"]["scale"], 32, dtype=torch.bfloat16),
                       r["mxfp8_qk_q"]["dequant_bf16"])
    assert torch.equal(OQ.mxfp8_v_dequant(f8(r["mxfp8_v_v"]["codes"]), r["mxfp8_v_v"]["scale"], 64, dtype=torch.bfloat16),
                       r["mxfp8_v_v"]["dequant_bf16"])
    ks, mean = OQ.smooth_k(k)
    assert torch.equal(ks, r["smooth_k"]["out"]) and ulp_close(mean, r["smooth_k"]["mean"], 2)
    qs, qm = OQ.group_mean_q(q, block_q=128)
    assert torch.equal(qs, r["group_mean_q128"]["out"]) and ulp_close(qm, r["group_mean_q128"]["qm"], 2)
    vs, va = OQ.smooth_v_per_block(v, block_s=64)
    assert torch.equal(vs, r["smooth_v64"]["out"]) and ulp_close(va, r["smooth_v64"]["alpha"], 2)
    qh, kh = OQ.apply_qk_hadamard(q, k, random_sign=True, seed=0)
    assert torch.equal(qh, r["hadamard"]["q"]) and torch.equal(kh, r["hadamard"]["k"])


def _k12_case_names(vec_path=FIXTURE):
    names = [f"d128/{n}" for n in C.K12_CASES] + [f"d64/{n}" for n in C.K12_CASES_D64]
    return names


def unpack_k12(vec, name):
    rec = vec["k12"][name]
    if "error" in rec:
        pytest.skip(f"the reference's own kernel failed for this case when the vectors were recorded: {rec['error'][:80]}")
    pool = vec["pool"]
    ops = [pool[k] for k in rec["ops"]]
    kw = {a: (pool[b] if tag == "T" else b) for a, (tag, b) in rec["kw"].items()}
    return ops, kw, rec


@pytest.mark.parametrize("name", _k12_case_names())
def test_streaming_kernel_restatement(vec, name):
    ops, kw, rec = unpack_k12(vec, name)
    res = k12_attention(
        ops[0].float(), ops[1].float(), ops[2].float(), ops[3],
        sm_scale=kw["sm_scale"], p_max_offset=kw["p_max_offset"], block_m=kw["block_m"], block_n=kw["block_n"],
        v_alpha=kw.get("v_alpha"), v_smooth_block=kw.get("v_smooth_block", 0),
        k_smooth=kw.get("k_smooth_bhsd"), qm=kw.get("qm_bhgd"), q_smooth_block=kw.get("q_smooth_block", 0),
        v_block_scale=kw.get("v_block_scale_bsh"), v_block_size=kw.get("v_block_size", 0),
        p_quant_mode=kw.get("p_quant_mode", "elementwise"), rowmax_est=kw.get("rowmax_est_bhs"),
        rowmax_init=kw.get("rowmax_init_bhs"),
        blasst_lambda=kw.get("blasst_lambda"), blasst_fill_mode=kw.get("blasst_fill_mode", "zero"),
        blasst_fill_alpha=kw.get("blasst_fill_alpha", 1.0), blasst_uta_bins=kw.get("blasst_uta_bins", 16),
        faithful=True, return_stats=kw.get("return_blasst_stats", False))
    if kw.get("return_blasst_stats", False):
        res, stats = res
        assert torch.equal(stats, rec["stats"]), name                        # every skip decision, bit for bit
        assert rec["skipped"] > 0
    over, cos = attention_report(res, rec["out"])
    assert cos >= 0.99999 and over <= ATT_FRAC, (name, cos, over)


@pytest.mark.parametrize("name", list(C.ENTRY_CASES))
def test_whole_entry_restatement(vec, name):
    s, h, d = C.ENTRY_SHAPE
    q, k, v = C.base_inputs(300, s, h, d)
    lab = vec["entry"]["labels"]
    cfg = QuantConfig(**C.ENTRY_CASES[name])
    got = OA.fake_quant_attention(q, k, v, cfg, faithful=True, out_fp32=True,
                                  q_labels=lab["q"].long() if cfg.q_kmeans_k is not None else None,
                                  v_labels=lab["v"].long() if cfg.v_kmeans_k is not None else None)
    over, cos = attention_report(got, vec["entry"][name]["out"])
    assert cos >= 0.99999 and over <= (ATT_FRAC if cfg.p_requant else ATT_FRAC_SDPA), (name, cos, over)
