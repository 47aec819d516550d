"""Generates the golden fixtures of this folder from the reference project.

Run once, in a container that has the reference checked out, with no GPU:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference package (with a stub for its un-vendored
``flash_kmeans`` dependency, which is only needed at import time) and calls
the parts of it that execute on CPU tensors:

* hadamard.py: ``_torch_hadamard_transform``, ``_cached_cpu_signs``
* attention.py: ``_estimate_rowmax_from_qm_k``, ``_fake_quant_attention_sdpa``,
  ``_preprocess`` / ``_fake_quant_attention_p_requant`` (orchestration only:
  the Triton kernels they call cannot run on CPU and are replaced, for the
  duration of the call, by the restatements under ``oracle/`` -- those fixtures
  therefore pin the glue, not the kernels)
* attention_triton.py: ``_parse_blasst_fill``
* the torch mirrors the reference's own tests compare its kernel with
  (tests/test_triton_attn.py: ``_torch_chunked_p_requant``,
  ``_torch_blasst_fill_reference``) -- these pin ``oracle/k12.py``.

Inputs are seeded random tensors; outputs are stored next to them.
"""
import importlib.util
import math
import os
import sys
import types

import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/reference")
REF = sys.argv[1]
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(REF, "src"))

stub = types.ModuleType("flash_kmeans")
stub.batch_kmeans_Euclid = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("stub"))
sys.modules["flash_kmeans"] = stub

import low_bit_fake_quant as ref                      # noqa: E402  (the reference package)
from low_bit_fake_quant import attention as ref_att   # noqa: E402
from low_bit_fake_quant import attention_triton as ref_k12  # noqa: E402
from low_bit_fake_quant import hadamard as ref_had    # noqa: E402
from low_bit_fake_quant import kmeans as ref_km       # noqa: E402

from oracle import api as OA                          # noqa: E402
from oracle import quant_ops as OQ                    # noqa: E402
from oracle.k12 import k12_attention                  # noqa: E402

spec = importlib.util.spec_from_file_location("ref_test_triton_attn", os.path.join(REF, "tests", "test_triton_attn.py"))
ref_tests = importlib.util.module_from_spec(spec)
spec.loader.exec_module(ref_tests)

out = {}

# ---- Hadamard ---------------------------------------------------------------
g = torch.Generator().manual_seed(11)
for d, dt in ((128, torch.bfloat16), (64, torch.float16)):
    x = torch.randn(3, 5, 2, d, generator=g).to(dt)
    y = ref_had._torch_hadamard_transform(x, scale=1.0 / math.sqrt(d))
    out[f"hadamard_d{d}"] = {"x": x, "y": y}
out["signs"] = {"h6_d128_s0": ref_had._cached_cpu_signs(6, 128, 0), "h3_d64_s7": ref_had._cached_cpu_signs(3, 64, 7)}

# ---- row-max estimate -------------------------------------------------------
qm = torch.randn(2, 4, 3, 64, generator=g)
kw = torch.randn(2, 512, 3, 64, generator=g).bfloat16()
out["rowmax_qm_k"] = {"qm": qm, "k": kw, "block_q": 128, "sm_scale": 0.125,
                      "y": ref_att._estimate_rowmax_from_qm_k(qm, kw, block_q=128, sm_scale=0.125, chunk_n=300)}

# ---- BLASST fill parser -----------------------------------------------------
cases = ["zero", None, "max", "max_a0.25", "mean", "mean_a1.5", "logn", "sample8", "sample8_a1.25", "thr",
         "thr_a0.25", "uta", "uta16_a1.5", "uta8", "uta4_a2"]
out["parse_fill"] = [(c, ref_k12._parse_blasst_fill(c, alpha=0.75, uta_bins=8)) for c in cases]

# ---- torch mirrors of the kernel from the reference's tests ------------------
torch.manual_seed(0)
B, H, S, D = 1, 2, 256, 128
q = torch.randn(B, H, S, D).bfloat16()
k = torch.randn(B, H, S, D).bfloat16()
vf = torch.randn(B, H, S, D).bfloat16()
v_scale = (vf.float().abs().amax(dim=-2) / 448.0).clamp_min(1e-6)
v_bf16 = (vf.float() / v_scale.unsqueeze(-2)).clamp(-448, 448).to(torch.float8_e4m3fn).to(torch.bfloat16)
y = ref_tests._torch_chunked_p_requant(q, k, v_bf16, v_scale, 1.0 / math.sqrt(D), 8, q_chunk=64)
out["mirror_elementwise"] = {"q": q, "k": k, "v": v_bf16, "v_scale": v_scale, "y": y}

torch.manual_seed(12)
B, H, S, D = 1, 1, 128, 64
u = torch.randn(D)
u = u / u.norm()
q = (u.view(1, 1, 1, D) + 0.01 * torch.randn(B, H, S, D)).bfloat16()
k = 0.05 * torch.randn(B, H, S, D)
k[:, :, :32, :] = 4.0 * u.view(1, 1, 1, D)
k = k.bfloat16()
v = torch.randn(B, H, S, D).bfloat16()
fills = {}
for mode in ["max_a0.25", "mean_a1.5", "logn", "sample8_a1.25", "thr_a0.25", "uta16_a1.5"]:
    fills[mode] = ref_tests._torch_blasst_fill_reference(
        q, k, v, torch.ones(B, H, D), sm_scale=1.0 / math.sqrt(D), p_max_offset=8, block_m=32, block_n=32,
        lam=0.8, fill_mode=mode)
out["mirror_blasst"] = {"q": q, "k": k, "v": v, "lam": 0.8, "fills": fills}

# ---- orchestration with the Triton kernels swapped for the restatements ------
def patch(mod):
    for name in ("fp8_block_quant", "fp8_block_dequant", "fp8_per_channel_quant", "fp8_per_channel_dequant",
                 "mxfp8_qk_quant", "mxfp8_qk_dequant", "mxfp8_v_quant", "mxfp8_v_dequant", "smooth_k",
                 "group_mean_q", "smooth_v_per_block"):
        setattr(mod, name, getattr(OQ, name))
    mod.apply_qk_hadamard = lambda q, k, random_sign=True, seed=0: (
        ref_had._torch_hadamard_transform(q * (ref_had._cached_cpu_signs(q.shape[2], q.shape[3], seed).view(1, 1, q.shape[2], q.shape[3]).to(q.dtype) if random_sign else 1), scale=1.0 / math.sqrt(q.shape[3])),
        ref_had._torch_hadamard_transform(k * (ref_had._cached_cpu_signs(k.shape[2], k.shape[3], seed).view(1, 1, k.shape[2], k.shape[3]).to(k.dtype) if random_sign else 1), scale=1.0 / math.sqrt(k.shape[3])))

patch(ref_att)

def k12_as_triton(q_bhsd, k_bhsd, v_bhsd_bf16, v_scale_bhd, **kw):
    res = k12_attention(q_bhsd.float(), k_bhsd.float(), v_bhsd_bf16.float(), v_scale_bhd,
                        sm_scale=kw["sm_scale"], p_max_offset=kw["p_max_offset"], block_m=kw["block_m"], block_n=kw["block_n"],
                        v_alpha=kw.get("v_alpha"), v_smooth_block=kw.get("v_smooth_block", 0),
                        k_smooth=kw.get("k_smooth_bhsd"), qm=kw.get("qm_bhgd"), q_smooth_block=kw.get("q_smooth_block", 0),
                        v_block_scale=kw.get("v_block_scale_bsh"), v_block_size=kw.get("v_block_size", 0),
                        p_quant_mode=kw.get("p_quant_mode", "elementwise"), rowmax_est=kw.get("rowmax_est_bhs"),
                        blasst_lambda=kw.get("blasst_lambda"), blasst_fill_mode=kw.get("blasst_fill_mode", "zero"),
                        blasst_fill_alpha=kw.get("blasst_fill_alpha", 1.0), blasst_uta_bins=kw.get("blasst_uta_bins", 16),
                        faithful=True)
    return res.to(torch.bfloat16)

ref_att.fake_quant_attention_triton = k12_as_triton

def fake_kmeans(t, *, n_clusters, max_iters=10, seed=0, chunk_tokens=4096):
    r = OA.kmeans_reorder_tokens(t, n_clusters=n_clusters, max_iters=max_iters, seed=seed)
    return ref_km.KMeansReorderResult(r.tensor_reordered, r.order, r.inverse_order, r.labels)

ref_att.q_kmeans_reorder = lambda q, n_clusters=32, max_iters=10, seed=0: fake_kmeans(q, n_clusters=n_clusters, max_iters=max_iters, seed=seed)
ref_att.v_kmeans_reorder = lambda v, n_clusters=32, max_iters=10, seed=0: fake_kmeans(v, n_clusters=n_clusters, max_iters=max_iters, seed=seed)

torch.manual_seed(5)
B, S, H, D = 1, 256, 2, 64
q = torch.randn(B, S, H, D).bfloat16()
k = (torch.randn(B, S, H, D) + 2.0 * torch.randn(1, 1, H, D)).bfloat16()
v = torch.randn(B, S, H, D).bfloat16()
glue = {"q": q, "k": k, "v": v, "cases": []}
cfgs = [
    dict(fp8_block_size=64, smoothing="off", q_kmeans_k=None, p_requant=False),
    dict(fp8_block_size=64, smoothing="full", q_kmeans_k=8, p_requant=False, v_smooth_mode="per_block", q_smooth_block_size=128),
    dict(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="elementwise"),
    dict(fp8_block_size=64, smoothing="full", q_kmeans_k=8, v_kmeans_k=8, v_smooth_mode="per_block",
         p_quant="dynamic", rowmax_mode="qm_k", q_smooth_block_size=128),
    dict(qk_quant="mxfp8", v_quant="mxfp8", smoothing="off", q_kmeans_k=None, qk_hadamard=True),
    dict(fp8_block_size=64, v_quant="fp8_block", smoothing="k_only", q_kmeans_k=None, p_quant="dynamic",
         blasst_lambda=1e-2, blasst_fill="uta16_a1.5"),
]
for kw in cfgs:
    cfg = ref.QuantConfig(**kw)
    qw, kw_, vw, qm_, va, qkm, vkm = ref_att._preprocess(q, k, v, cfg)
    sm = 1.0 / math.sqrt(D)
    if cfg.p_requant:
        o = ref_att._fake_quant_attention_p_requant(qw, kw_, vw, qm_, va, qkm, cfg, sm, torch.bfloat16)
    else:
        o = ref_att._fake_quant_attention_sdpa(qw, kw_, vw, qm_, va, cfg, sm, torch.bfloat16).to(torch.bfloat16)
    if qkm is not None:
        inv = qkm.inverse_order
        ob = o.permute(0, 2, 1, 3).reshape(B * H, S, D)
        o = torch.gather(ob, 1, inv.unsqueeze(-1).expand(-1, -1, D)).reshape(B, H, S, D).permute(0, 2, 1, 3).contiguous()
    glue["cases"].append({"cfg": kw, "out": o})
out["glue"] = glue

torch.save(out, os.path.join(HERE, "reference_cpu_vectors.pt"))
print("wrote", os.path.join(HERE, "reference_cpu_vectors.pt"), os.path.getsize(os.path.join(HERE, "reference_cpu_vectors.pt")), "bytes")
