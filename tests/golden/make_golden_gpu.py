"""Records golden vectors from the reference project's OWN Triton kernels, run on a GPU.

Needs: a CUDA device, Triton, and the reference package staged by ``python oracle/make_ref.py /path/to/reference``.

    python tests/golden/make_golden_gpu.py [out.pt]          (default: tests/golden/reference_gpu_vectors.pt)

What it records (all inputs are the seeded tensors of ``ref_gpu_cases.py``, stored beside the outputs):

* ``quant``: codes and scales of the reference's four quantizers (quant_triton.py:61-77, 163-176, 255-271,
  354-369), its de-quantizers, its three smoothing kernels (preprocess.py:38-57, 135-193) and its Hadamard rotation
  (hadamard.py:77-117) -- the pins for ``oracle/quant_ops.py`` and for ``csrc/quant.cu`` / ``csrc/preprocess.cu``;
* ``k12``: outputs (and BLASST stats) of direct launches of the streaming kernel (attention_triton.py:410-671) in
  every P / V / row-max / BLASST mode, with the exact operands the reference's glue built for them -- the pins for
  ``oracle/k12.py`` and for the BF16-operand instantiation of the CUDA kernel;
* ``entry``: outputs of ``fake_quant_attention`` (attention.py:706-806) for whole configurations, k-means labels
  injected (the reference's third-party k-means is not available; the labels are stored);
* ``stats``: mismatch rates at larger sizes (quantizer codes and scales of the reference vs this library vs the
  IEEE-division formula) and attention parity figures (this library in both operand conventions vs the reference).
"""
import hashlib
import os
import sys
import traceback

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "low-bit-attention-fake-quant_b200"), HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

import ref_gpu_cases as C                 # noqa: E402
from oracle import ref_gpu                # noqa: E402
from oracle import api as OA              # noqa: E402

ref = ref_gpu.load()
if ref is None or not torch.cuda.is_available():
    raise SystemExit("make_golden_gpu.py needs CUDA, Triton and the staged reference (python oracle/make_ref.py <reference>)")
import low_bit_fake_quant as ours         # noqa: E402

dev = torch.device("cuda:0")
out = {"errors": {}, "versions": {"torch": torch.__version__, "triton": __import__("triton").__version__,
                                  "gpu": torch.cuda.get_device_name(0)}}
pool = {}


def keep(t):
    """Store a tensor once (by content) and return its key."""
    t = t.detach().cpu().contiguous()
    raw = t.view(torch.uint8) if t.dtype != torch.bool else t.to(torch.uint8)
    key = hashlib.sha1(raw.numpy().tobytes() + str((t.dtype, tuple(t.shape))).encode()).hexdigest()[:16]
    pool.setdefault(key, t)
    return key


def u8(t):
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


def section(name):
    def deco(fn):
        try:
            out[name] = fn()
            print(f"[golden] {name}: ok", flush=True)
        except Exception:                                  # keep going: one failed section must not lose the others
            out["errors"][name] = traceback.format_exc()
            print(f"[golden] {name}: FAILED\n{out['errors'][name]}", flush=True)
        return fn
    return deco


@section("quant")
def _quant():
    res = {}
    for (s, h, d) in C.OP_SHAPES:
        q, k, v = (t.to(dev) for t in C.base_inputs(100 + d, s, h, d))
        r = {"shape": (s, h, d), "seed": 100 + d}
        for nm, fn, x, kw in (("fp8_block64_q", ref.fp8_block_quant, q, dict(block_s=64)),
                              ("fp8_block128_k", ref.fp8_block_quant, k, dict(block_s=128)),
                              ("fp8_channel_v", ref.fp8_per_channel_quant, v, {}),
                              ("mxfp8_qk_q", ref.mxfp8_qk_quant, q, dict(block_d=32)),
                              ("mxfp8_v_v", ref.mxfp8_v_quant, v, dict(block_s=64))):
            c, sc = fn(x, **kw)
            r[nm] = {"codes": u8(c).cpu(), "scale": sc.cpu()}
        c, sc = ref.fp8_block_quant(q, block_s=64)
        r["fp8_block64_q"]["dequant_bf16"] = ref.fp8_block_dequant(c, sc, block_s=64, dtype=torch.bfloat16).cpu()
        c, sc = ref.fp8_per_channel_quant(v)
        r["fp8_channel_v"]["dequant_bf16"] = ref.fp8_per_channel_dequant(c, sc, dtype=torch.bfloat16).cpu()
        c, sc = ref.mxfp8_qk_quant(q, block_d=32)
        r["mxfp8_qk_q"]["dequant_bf16"] = ref.mxfp8_qk_dequant(c, sc, block_d=32, dtype=torch.bfloat16).cpu()
        c, sc = ref.mxfp8_v_quant(v, block_s=64)
        r["mxfp8_v_v"]["dequant_bf16"] = ref.mxfp8_v_dequant(c, sc, block_s=64, dtype=torch.bfloat16).cpu()
        for dt in (torch.float16, torch.float32):
            c, sc = ref.fp8_block_quant(q.to(dt), block_s=64)
            r[f"fp8_block64_q_{str(dt).split('.')[-1]}"] = {"codes": u8(c).cpu(), "scale": sc.cpu()}
        ks, mean = ref.smooth_k(k)
        r["smooth_k"] = {"out": ks.cpu(), "mean": mean.cpu()}
        qs, qm = ref.group_mean_q(q, block_q=128)
        r["group_mean_q128"] = {"out": qs.cpu(), "qm": qm.cpu()}
        vs, va = ref.smooth_v_per_block(v, block_s=64)
        r["smooth_v64"] = {"out": vs.cpu(), "alpha": va.cpu()}
        qh, kh = ref.apply_qk_hadamard(q, k, random_sign=True, seed=0)
        r["hadamard"] = {"q": qh.cpu(), "k": kh.cpu()}
        res[f"d{d}"] = r
    return res


@section("k12")
def _k12():
    res = {}
    from ref_low_bit_fake_quant.attention_triton import fake_quant_attention_triton as ref_k12
    for (s, h, d) in C.OP_SHAPES:
        names = list(C.K12_CASES) if d == 128 else list(C.K12_CASES_D64)
        q, k, v = (t.to(dev) for t in C.base_inputs(200 + d, s, h, d))
        for nm in names:
            spec = C.K12_CASES[nm]
            ops, kw = C.build_k12_operands(ref, q, k, v, spec, sm_scale=C.sm_scale_for(d))
            try:
                got = ref_k12(*ops, **kw)
            except Exception as e:                         # e.g. a Triton compiler failure for one instantiation
                res[f"d{d}/{nm}"] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
                print(f"[golden]   k12 d{d}/{nm} FAILED in the reference: {type(e).__name__}", flush=True)
                continue
            stats = None
            if isinstance(got, tuple):
                got, stats = got
            torch.cuda.synchronize()
            rec = {"ops": [keep(t) for t in ops],
                   "kw": {a: (("T", keep(b)) if torch.is_tensor(b) else ("V", b)) for a, b in kw.items()},
                   "out": got.cpu(), "stats": stats.cpu() if stats is not None else None}
            if stats is not None:
                rec["skipped"] = float(stats[..., 0].sum())
            res[f"d{d}/{nm}"] = rec
            print(f"[golden]   k12 d{d}/{nm} done" + (f" (skipped {rec['skipped']:.0f})" if stats is not None else ""), flush=True)
    return res


def run_entry(cfg_kwargs, q, k, v, labels):
    cfg_r = ref.QuantConfig(**cfg_kwargs)
    if labels:
        ref_gpu.inject_labels(*labels)
    return ref.fake_quant_attention(q, k, v, cfg_r)


@section("entry")
def _entry():
    res = {}
    s, h, d = C.ENTRY_SHAPE
    q, k, v = (t.to(dev) for t in C.base_inputs(300, s, h, d))
    ql = ours.kmeans.kmeans_labels(q, n_clusters=8).cpu()
    vl = ours.kmeans.kmeans_labels(v, n_clusters=8).cpu()
    res["labels"] = {"q": ql.to(torch.int16), "v": vl.to(torch.int16)}
    for nm, kw in C.ENTRY_CASES.items():
        labels = []
        if kw.get("q_kmeans_k") is not None:
            labels.append(ql)
        if kw.get("v_kmeans_k") is not None:
            labels.append(vl)
        o = run_entry(kw, q, k, v, labels)
        torch.cuda.synchronize()
        res[nm] = {"out": o.cpu()}
        print(f"[golden]   entry {nm} done", flush=True)
    return res


def bench_like(seed, s, h, d):
    g = torch.Generator().manual_seed(seed)
    scale = torch.ones(d)
    scale[torch.tensor([5, 37, 70, 101]) % d] = 10.0
    q = torch.randn(1, s, h, d, generator=g) * scale
    k = torch.randn(1, s, h, d, generator=g) * scale + 3.0 * torch.randn(1, 1, h, d, generator=g)
    v = torch.randn(1, s, h, d, generator=g)
    return q.bfloat16().to(dev), k.bfloat16().to(dev), v.bfloat16().to(dev)


def mismatch(a, b):
    a, b = u8(a), u8(b)
    return float((a != b).float().mean())


@section("stats_quant")
def _stats_quant():
    """Reference Triton quantizers vs this library vs the IEEE-division formula, 4.2 M elements per tensor."""
    st = {}
    q, k, v = bench_like(7, 4096, 8, 128)

    def ieee_block(x, blk):
        b, s, h, d = x.shape
        xf = x.float().view(b, s // blk, blk, h, d)
        amax = xf.abs().amax(dim=(2, 4)).clamp_min(1e-4)
        sc = amax / 448.0
        codes = (xf / sc[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(b, s, h, d)
        return codes, sc

    rc, rs = ref.fp8_block_quant(q, block_s=64)
    oc, os_ = ours.fp8_block_quant(q, block_s=64)
    ic, is_ = ieee_block(q, 64)
    st["fp8_block64"] = {"codes_ref_vs_ours": mismatch(rc, oc), "codes_ref_vs_ieee": mismatch(rc, ic),
                         "codes_ours_vs_ieee": mismatch(oc, ic),
                         "scale_ref_vs_ours": float((rs != os_).float().mean()), "scale_ref_vs_ieee": float((rs != is_).float().mean()),
                         "scale_max_rel": float(((rs - os_).abs() / os_).max())}
    rc, rs = ref.fp8_per_channel_quant(v)
    oc, os_ = ours.fp8_per_channel_quant(v)
    st["fp8_channel"] = {"codes_ref_vs_ours": mismatch(rc, oc), "scale_ref_vs_ours": float((rs != os_).float().mean()),
                         "scale_max_rel": float(((rs - os_).abs() / os_).max())}
    rc, rs = ref.mxfp8_qk_quant(q, block_d=32)
    oc, os_ = ours.mxfp8_qk_quant(q, block_d=32)
    st["mxfp8_qk"] = {"codes_ref_vs_ours": mismatch(rc, oc), "scale_ref_vs_ours": float((rs != os_).float().mean())}
    rc, rs = ref.mxfp8_v_quant(v, block_s=64)
    oc, os_ = ours.mxfp8_v_quant(v, block_s=64)
    st["mxfp8_v"] = {"codes_ref_vs_ours": mismatch(rc, oc), "scale_ref_vs_ours": float((rs != os_).float().mean())}
    a, am = ref.smooth_k(k)
    b_, bm = ours.smooth_k(k)
    st["smooth_k"] = {"out_ref_vs_ours": float((a != b_).float().mean()), "mean_ref_vs_ours": float((am != bm).float().mean()),
                      "mean_max_abs": float((am - bm).abs().max())}
    a, am = ref.group_mean_q(q, block_q=256)
    b_, bm = ours.group_mean_q(q, block_q=256)
    st["group_mean_q"] = {"out_ref_vs_ours": float((a != b_).float().mean()), "mean_ref_vs_ours": float((am != bm).float().mean()),
                          "mean_max_abs": float((am - bm).abs().max())}
    a, am = ref.smooth_v_per_block(v, block_s=64)
    b_, bm = ours.smooth_v_per_block(v, block_s=64)
    st["smooth_v"] = {"out_ref_vs_ours": float((a != b_).float().mean()), "mean_ref_vs_ours": float((am != bm).float().mean()),
                      "mean_max_abs": float((am - bm).abs().max())}
    a, a2 = ref.apply_qk_hadamard(q, k, random_sign=True, seed=0)
    b_, b2 = ours.apply_qk_hadamard(q, k, random_sign=True, seed=0)
    st["hadamard"] = {"q_ref_vs_ours": float((a != b_).float().mean()), "k_ref_vs_ours": float((a2 != b2).float().mean())}
    print("[golden]   stats_quant", st, flush=True)
    return st


@section("stats_attention")
def _stats_attention():
    """This library, in both operand conventions, against the reference's own path at S = 2048 (k-means labels shared)."""
    st = {}
    s, h, d = 2048, 2, 128
    q, k, v = bench_like(11, s, h, d)
    sdpa = ours.reference_attention(q, k, v).float().cpu()
    stacks = {
        "k_smooth_static": dict(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="elementwise"),
        "full_dynamic": dict(fp8_block_size=64, smoothing="full", q_kmeans_k=32, q_smooth_block_size=256, v_kmeans_k=64,
                             v_smooth_mode="per_block", v_smooth_block_size=64, p_quant="dynamic", rowmax_mode="qm_k"),
        "mxfp8_hadamard": dict(qk_quant="mxfp8", v_quant="mxfp8", mxfp8_block_size=32, v_mxfp8_block_size=64, qk_hadamard=True,
                               smoothing="off", q_kmeans_k=None, p_quant="auto"),
        "blasst_mean_dynamic": dict(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="dynamic",
                                    blasst_lambda=1e-2, blasst_fill="mean_a1.5"),
    }
    for nm, kw in stacks.items():
        labels, okw = [], {}
        if kw.get("q_kmeans_k") is not None:
            ql = ours.kmeans.kmeans_labels(q, n_clusters=kw["q_kmeans_k"])
            labels.append(ql)
            okw["_q_labels"] = ql
        if kw.get("v_kmeans_k") is not None:
            vl = ours.kmeans.kmeans_labels(v, n_clusters=kw["v_kmeans_k"])
            labels.append(vl)
            okw["_v_labels"] = vl
        r = run_entry(kw, q, k, v, labels).float().cpu()
        cfg = ours.QuantConfig(**kw)
        rec = {"ref_vs_sdpa": OA.compute_metrics(r, sdpa)}
        rms = float(r.pow(2).mean().sqrt())
        for mode, extra in (("fp8_codes", {}), ("reference_operands", {"_reference_operands": True})):
            try:
                o = ours.fake_quant_attention(q, k, v, cfg, **okw, **extra).float().cpu()
            except NotImplementedError as e:
                rec[mode] = {"not_implemented": str(e)}
                continue
            m = OA.compute_metrics(o, r)
            m["max_abs_over_rms"] = m["max_abs"] / rms
            err = (o - r).abs()
            ulp = r.abs().clamp_min(1e-30).log2().floor().exp2() * 2.0 ** -7        # one BF16 ulp of the reference value
            m["frac_over_1ulp_plus_tol"] = float((err > ulp + 2e-3 * rms).float().mean())
            m["vs_sdpa"] = OA.compute_metrics(o, sdpa)
            rec[mode] = m
        st[nm] = rec
        print(f"[golden]   stats_attention {nm}: {rec}", flush=True)
    return st


out["pool"] = pool
dst = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_gpu_vectors.pt")
os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
torch.save(out, dst)
print("[golden] wrote", dst, os.path.getsize(dst), "bytes; errors:", list(out["errors"]))
