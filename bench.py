#!/usr/bin/env python
"""Benchmark of the fake-quant attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one call of ``low_bit_fake_quant.fake_quant_attention`` on the
Wan-14B self-attention shape (B=1, H=40, S=32760 padded to 32768 by the
reference hook's rule, D=128, BF16) with the ``full_dynamic`` stack -- Q k-means
32 + V k-means 64 with K co-permuted, full Q/K smoothing, per-block V
smoothing, fp8_block 64 Q/K, fp8_channel V, dynamic P, qm_k estimated row max,
64x64 blocks: k-means, smoothing, quantizers and the attention kernel
together. The ``k_smooth_static`` stack of the same shape is timed in the same
run and reported under ``config.also``. With N > 1 (launched under torchrun)
every rank runs one such problem on its own GPU (weak scaling, global batch =
N: ``value``); the same run also times ONE problem partitioned over the ranks,
40/N heads each (``strong_scaling``). The path has no collective.

Printed JSON (rank 0): throughput in TFLOP/s with the algorithmic flop count
4*B*H*Sq*Sk*D on the unpadded shape; ``e2e`` is the same call fed from pinned
host buffers with the result copied back; ``roofline`` describes the
attention kernel against the dense-FP8 tensor peak; ``parity`` compares one
head of the very tensors that were timed with the CPU oracle; ``cpu_baseline``
is the CPU restatement of the reference timed on a bounded sample.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "low-bit-attention-fake-quant_b200"))

import torch  # noqa: E402

H_FULL, S_REAL, D_HEAD = 40, 32760, 128

WORKLOADS = {
    # name: (QuantConfig kwargs, batch)
    "wan14b_self_attn_k_smooth_static": (dict(
        qk_quant="fp8_block", v_quant="fp8_channel", q_smooth_block_size=256, fp8_block_size=64, p_requant=True,
        p_requant_block_m=64, p_requant_block_n=64, smoothing="k_only", q_kmeans_k=None, v_smooth_mode="off",
        v_kmeans_k=None, p_quant="elementwise", rowmax_mode="online"), 1),
    "wan14b_self_attn_full_dynamic": (dict(
        qk_quant="fp8_block", v_quant="fp8_channel", q_smooth_block_size=256, fp8_block_size=64, p_requant=True,
        p_requant_block_m=64, p_requant_block_n=64, smoothing="full", q_kmeans_k=32, v_smooth_mode="per_block",
        v_smooth_block_size=64, v_kmeans_k=64, p_quant="dynamic", rowmax_mode="qm_k"), 1),
    # the other two stacks of the benchmark list (mxfp8 + Hadamard; BLASST skip / fill on video-like tokens): parity-test
    # cases first, timed here for the record
    "wan14b_self_attn_mxfp8_hadamard": (dict(
        qk_quant="mxfp8", v_quant="mxfp8", mxfp8_block_size=32, v_mxfp8_block_size=64, qk_hadamard=True, p_requant=True,
        p_requant_block_m=64, p_requant_block_n=64, smoothing="off", q_kmeans_k=None, v_smooth_mode="off",
        v_kmeans_k=None, p_quant="auto", rowmax_mode="online"), 1),
    # the cross-attention shape of the same stack (32760 video queries over 512 text keys): an extension with no
    # counterpart in the reference, whose hook sends cross-attention to plain SDPA; device-resident timing only
    "wan14b_cross_attn_mxfp8_hadamard": (dict(
        qk_quant="mxfp8", v_quant="mxfp8", mxfp8_block_size=32, v_mxfp8_block_size=64, qk_hadamard=True, p_requant=True,
        p_requant_block_m=64, p_requant_block_n=64, smoothing="off", q_kmeans_k=None, v_smooth_mode="off",
        v_kmeans_k=None, p_quant="auto", rowmax_mode="online"), 1, 512),
    "wan14b_video_blasst_mean_1e-2": (dict(
        qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, p_requant=True, p_requant_block_m=64,
        p_requant_block_n=64, smoothing="k_only", q_kmeans_k=None, v_smooth_mode="off", v_kmeans_k=None,
        p_quant="dynamic", rowmax_mode="online", blasst_lambda=1e-2, blasst_fill="mean_a1.5"), 2),
}
VIDEO_GRID = (21, 30, 52)       # (t, h, w) of the 32760 latent tokens, flattened t-major
# the stack the project's target is stated on; the other stack of the same shape is timed beside it
DEFAULT_WORKLOAD = "wan14b_self_attn_full_dynamic"
ALSO = {"wan14b_self_attn_full_dynamic": "wan14b_self_attn_k_smooth_static",
        "wan14b_self_attn_k_smooth_static": "wan14b_self_attn_full_dynamic"}


def make_video_inputs(batch, heads, seq, dim, seed, device, dtype=torch.bfloat16):
    """Spatially local stand-in for video tokens: Q / K = a sum of 16 random low-frequency sinusoids over the (t, h, w)
    grid with random per-channel phases + N(0, 0.3) noise, so that attention mass is local; V ~ N(0, 1)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    t, hh, w = VIDEO_GRID
    idx = torch.arange(seq)
    pos = torch.stack((idx // (hh * w) / t, (idx // w) % hh / hh, idx % w / w), dim=1).to(device)       # (S, 3) in [0, 1)
    gd = torch.Generator(device=device).manual_seed(seed)
    out = []
    for _ in range(2):
        freq = (torch.randint(1, 4, (16, 3), generator=g).float() * 2 * math.pi).to(device)             # 16 waves
        x = torch.zeros(batch, seq, heads, dim, device=device)
        for f in range(16):
            phase = (2 * math.pi * torch.rand(1, 1, heads, dim, generator=g)).to(device)
            x += torch.sin((pos @ freq[f]).view(1, seq, 1, 1) + phase) * 0.5
        x += 0.3 * torch.randn(batch, seq, heads, dim, generator=gd, device=device)
        out.append(x.to(dtype))
    v = torch.randn(batch, seq, heads, dim, generator=gd, device=device).to(dtype)
    return out[0], out[1], v


def make_inputs(batch, heads, seq, dim, seed, device, dtype=torch.bfloat16):
    """Seeded synthetic stand-in for a Wan2.1 layer's Q/K/V: N(0,1) with 4 of the
    128 channels scaled x10, K shifted by a per-channel mean ~ N(0,3), V ~ N(0,1)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    scale = torch.ones(dim)
    scale[torch.tensor([5, 37, 70, 101]) % dim] = 10.0
    kmean = 3.0 * torch.randn(1, 1, heads, dim, generator=g)
    gd = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(batch, seq, heads, dim, generator=gd, device=device) * scale.to(device)
    k = torch.randn(batch, seq, heads, dim, generator=gd, device=device) * scale.to(device) + kmean.to(device)
    v = torch.randn(batch, seq, heads, dim, generator=gd, device=device)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def pad_like_hook(q, k, v, cfg):
    """Pad S up to the lcm of the block sizes: Q rows zero, K/V replicate the last row
    (the policy of the reference's Wan hook, bench/wan_attention_hook.py:253-294)."""
    from low_bit_fake_quant.hook import pad_qkv
    qp, kp, vp, pad = pad_qkv(q, k, v, cfg)
    return qp.contiguous(), kp.contiguous(), vp.contiguous(), pad


def blasst_skip_ratios(qp, kp, vp, cfg, tile_predicate=False):
    """Row-skip and whole-program skip ratios from the kernel's stats tensor, computed the way the reference's BLASST
    evaluation does (bench/eval_blasst_quant.py:216-227), and the share of (128-row tile, key block) pairs the kernel
    did no work for (its own counter; zero fill only). One extra call, outside the timed region."""
    import low_bit_fake_quant as fq
    from low_bit_fake_quant.attention import _fake_quant_attention_p_requant
    k_work = fq.smooth_k(kp)[0] if cfg.smoothing != "off" else kp
    elided = torch.zeros(1, dtype=torch.int64, device=qp.device)
    _, stats = _fake_quant_attention_p_requant(qp, k_work, vp, None, None, None, cfg, 1.0 / math.sqrt(qp.shape[-1]),
                                               qp.dtype, return_stats=True, blasst_tile_predicate=tile_predicate,
                                               blasst_elided=elided)
    b, s, h, _ = qp.shape
    pairs = b * h * ((s + 127) // 128) * ((s + cfg.p_requant_block_n - 1) // cfg.p_requant_block_n)
    skipped, total = float(stats[..., 0].sum().item()), float(stats[..., 1].sum().item())
    tiles = stats[..., 1].gt(0)
    tile_skipped = float((stats[..., 0] == stats[..., 1]).logical_and(tiles).sum().item())
    return {"row_skip_ratio": skipped / total if total > 0 else 0.0,
            "tile_skip_ratio": tile_skipped / float(tiles.sum().item()) if tiles.any() else 0.0,
            "skipped_row_blocks": skipped, "total_row_blocks": total,
            "elided_tile_blocks": int(elided.item()), "elided_tile_block_ratio": float(elided.item()) / pairs,
            "tile_predicate": bool(tile_predicate)}


def load_traffic_table():
    """DRAM bytes per attention launch measured by ncu (profiles/dram_traffic.json): small 4-head captures, scaled
    here by heads (each head's traffic is independent)."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def verify_one_head(qp, kp, vp, cfg, head=0, reference_operands=False):
    """Parity of the timed inputs themselves: one head of the padded Q / K / V through the library (same k-means
    labels injected on both sides) against the CPU oracle -- first in the convention the launched kernel implements
    (e4m3 codes multiplied directly, scales in FP32 around the MMA; or, with ``--reference-operands``, the
    reference's BF16 de-quantised operands), which is the parity claim and is held to the tests' bound, then, for
    the code path, the distance to the reference's BF16-operand convention (the reference's own BF16 rounding of
    its operands, amplified by the softmax: a property of multiplying real FP8 codes) -- plus the MSE / cosine of
    each against BF16 SDPA. Outside every timed region."""
    import low_bit_fake_quant as fq
    from low_bit_fake_quant import _lib as L
    from low_bit_fake_quant.kmeans import kmeans_labels
    from oracle import api as OA
    from oracle import quant_ops as OQ

    dev = qp.device
    OQ.set_reciprocal(lambda t: L.rcp_approx(t, device=dev))          # the oracle divides as the GPU does
    q1, k1, v1 = (t[:, :, head:head + 1].contiguous() for t in (qp, kp, vp))
    kw, okw = {}, {}
    if cfg.q_kmeans_k is not None:
        kw["_q_labels"] = kmeans_labels(q1, n_clusters=cfg.q_kmeans_k, max_iters=cfg.q_kmeans_iters, seed=cfg.q_kmeans_seed)
        okw["q_labels"] = kw["_q_labels"].cpu().long()
    if cfg.v_kmeans_k is not None:
        kw["_v_labels"] = kmeans_labels(v1, n_clusters=cfg.v_kmeans_k, max_iters=cfg.v_kmeans_iters, seed=cfg.v_kmeans_seed)
        okw["v_labels"] = kw["_v_labels"].cpu().long()
    got = fq.fake_quant_attention(q1, k1, v1, cfg, _debug_fp32=True, _reference_operands=reference_operands, **kw).float().cpu()
    p_bf16 = L.lib().lbfq_attention_last_variant() == 1 and cfg.p_requant
    sdpa = fq.reference_attention(q1, k1, v1).float().cpu()
    torch.set_num_threads(os.cpu_count() or 1)
    qc, kc, vc = q1.cpu(), k1.cpu(), v1.cpu()
    t0 = time.perf_counter()
    if reference_operands:
        own = OA.fake_quant_attention(qc, kc, vc, cfg, faithful=True, out_fp32=True, **okw)
    else:
        own = OA.fake_quant_attention(qc, kc, vc, cfg, faithful=False, out_fp32=True, p_bf16=p_bf16, **okw)
    dt = time.perf_counter() - t0
    # the rule of oracle.api.parity_report, with the head's S x S softmax taken in row chunks: rows over 2e-3 x RMS
    # must stay within what one e4m3 code step of their largest P value can move them (a BF16 ulp of it is less), and be few
    rms = float(own.double().pow(2).mean().sqrt())
    row_err = (got - own).abs().amax(dim=-1)[0, :, 0]
    qf, kf = qc.float()[0, :, 0], kc.float()[0, :, 0]
    w_max = torch.empty(qf.shape[0])
    for r0 in range(0, qf.shape[0], 4096):
        w_max[r0:r0 + 4096] = torch.softmax((qf[r0:r0 + 4096] @ kf.t()) / math.sqrt(qf.shape[-1]), dim=-1).amax(dim=-1)
    tol = 2e-3 * rms
    flip_bound = tol + 2.0 * 0.125 * (2.0 * w_max).clamp_max(1.0) * vc.float().abs().max().item()
    a64, b64 = got.double().flatten(), own.double().flatten()
    rep = {"cosine": float(torch.dot(a64, b64) / (a64.norm() * b64.norm())), "max_abs_over_rms": float((a64 - b64).abs().max()) / rms,
           "flip_row_fraction": float((row_err > tol).float().mean()), "rows_over_flip_bound": int((row_err > flip_bound).sum())}
    ok = rep["cosine"] >= 0.99999 and rep["rows_over_flip_bound"] == 0 and rep["flip_row_fraction"] <= 0.01
    out = {"sample": f"head {head} of the timed tensors, S={qp.shape[1]}",
           "kernel_convention": "reference BF16 operands" if reference_operands else "e4m3 codes multiplied directly, scales in FP32",
           "vs_oracle_in_kernel_convention": {"cosine": rep["cosine"], "max_abs_over_rms": rep["max_abs_over_rms"],
                                              "rows_with_a_rounding_flip": rep["flip_row_fraction"],
                                              "rows_over_the_flip_bound": rep["rows_over_flip_bound"],
                                              "within_bound": bool(ok),
                                              "bound": "cosine >= 0.99999, max-abs <= 2e-3 x RMS outside rows where one P value on a "
                                                       "rounding boundary took the neighbouring e4m3 code or, in the scaled P modes, the "
                                                       "neighbouring BF16 value (<= 1 % of the rows, each within the single-flip bound)"},
           "mse_vs_sdpa": OA.compute_metrics(got, sdpa)["mse"], "mse_vs_sdpa_oracle": OA.compute_metrics(own, sdpa)["mse"],
           "oracle_seconds": dt}
    if not reference_operands:
        ref_conv = OA.fake_quant_attention(qc, kc, vc, cfg, faithful=True, out_fp32=True, **okw)
        r64 = ref_conv.double().flatten()
        rms = float(r64.pow(2).mean().sqrt())
        out["distance_to_reference_bf16_operand_convention"] = {
            "cosine": float(torch.dot(a64, r64) / (a64.norm() * r64.norm())), "max_abs_over_rms": float((a64 - r64).abs().max()) / rms,
            "mse_vs_sdpa_reference_convention": OA.compute_metrics(ref_conv, sdpa)["mse"],
            "note": "the reference rounds its de-quantised operands to BF16 before multiplying; FP8 MMAs multiply the codes "
                    "exactly. --reference-operands runs the reference's convention itself"}
    return out


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        return float(pk["bf16_tflops"]), float(pk["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0, "fallback"


def cpu_oracle_sample(cfg_kwargs, seq=4096, heads=1, steps=1, seed=0):
    """Time the CPU restatement of the reference path on a bounded sample of the
    workload (same distributions and config, `heads` heads x `seq` tokens)."""
    from low_bit_fake_quant.config import QuantConfig
    from oracle import api as OA
    cfg = QuantConfig(**cfg_kwargs)
    q, k, v = make_inputs(1, heads, seq, D_HEAD, seed, "cpu")
    OA.fake_quant_attention(q[:, :512], k[:, :512], v[:, :512], cfg)           # warm the thread pool
    t0 = time.perf_counter()
    for _ in range(steps):
        OA.fake_quant_attention(q, k, v, cfg, faithful=True)
    dt = (time.perf_counter() - t0) / steps
    flops = 4.0 * heads * seq * seq * D_HEAD
    return flops / dt / 1e12, dt


def run_reference_arm(args, workload, cfg_kwargs):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    seq, heads = 32768, 1                      # the sample the `cpu_baseline` leg of the other arm times
    vals = []
    for i in range(args.warmup + args.steps):
        tf, dt = cpu_oracle_sample(cfg_kwargs, seq=seq, heads=heads, steps=1, seed=i)
        if i >= args.warmup:
            vals.append((tf, dt))
    tf = sum(v[0] for v in vals) / len(vals)
    ms = 1e3 * sum(v[1] for v in vals) / len(vals)
    sample = f"{heads} head x S={seq} of the workload per step, oracle port (reference-faithful BF16 operand convention)"
    line = {
        "impl": "reference", "metric": "fused FP8 fake-quant attn TFLOP/s at 40x32760x128", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (simulated in fp32/bf16 on CPU)", "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--heads", type=int, default=H_FULL, help="heads per GPU (smaller values are for profiling runs only)")
    ap.add_argument("--seq", type=int, default=S_REAL)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the second timed stack (config.also)")
    ap.add_argument("--no-verify", action="store_true", help="skip the one-head parity check against the CPU oracle")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the one-problem-over-N-ranks partition")
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=None,
                    help="heads per pipelined chunk of the host-buffer entry (default: the entry's own choice)")
    ap.add_argument("--e2e-chunks", default=None,
                    help="the host-buffer entry's chunk sizes in heads, in order (e.g. 4,8,12,12,4); overrides the entry's own schedule")
    ap.add_argument("--reference-operands", action="store_true",
                    help="run path B on the reference's own BF16 operands (BF16 MMAs) instead of the FP8 codes; not the headline")
    ap.add_argument("--blasst-lambda", type=float, default=None, help="override the BLASST threshold of a BLASST workload")
    ap.add_argument("--blasst-fill", default=None, help="override the BLASST fill of a BLASST workload (zero, mean_a1.5, uta16_a1.5 ...)")
    ap.add_argument("--blasst-tile-predicate", action="store_true",
                    help="BLASST drops a key block only when all rows of a 128-row tile agree (the predicate of the "
                         "reference's simulator) instead of row by row; zero fill")
    ap.add_argument("--blasst-sweep", action="store_true",
                    help="BLASST workloads: also time the grid lambda in {1e-4, 1e-3, 1e-2} x fill in {zero, mean_a1.5, "
                         "uta16_a1.5} on the same tensors (config.blasst_sweep)")
    ap.add_argument("--brick", default=None,
                    help="ts,hs,ws: take the video workload's tokens brick by brick over its (21, 30, 52) grid (the reference's "
                         "space-time block reorder); the permutation of Q / K / V and of the result is inside the timed step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    cfg_kwargs, batch = WORKLOADS[args.workload][:2]
    seq_k = WORKLOADS[args.workload][2] if len(WORKLOADS[args.workload]) > 2 else None     # cross-attention: keys
    if cfg_kwargs.get("blasst_lambda") is not None:
        cfg_kwargs = dict(cfg_kwargs)
        if args.blasst_lambda is not None:
            cfg_kwargs["blasst_lambda"] = args.blasst_lambda
        if args.blasst_fill is not None:
            cfg_kwargs["blasst_fill"] = args.blasst_fill

    if args.impl == "reference":
        run_reference_arm(args, args.workload, cfg_kwargs)
        return

    import low_bit_fake_quant as fq
    from low_bit_fake_quant import _lib as L
    from low_bit_fake_quant import attention_triton as K12
    from low_bit_fake_quant.config import QuantConfig
    from low_bit_fake_quant.sharding import attention_on_shard, slab_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the shipped path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group(backend="nccl", device_id=dev)
        # bring the communicator up now, before any of the library's kernels is in flight: its set-up (peer
        # mappings, NVLS binding) otherwise runs under the first barrier, concurrently with the warm-up launches
        dist.all_reduce(torch.zeros(1, device=dev))
        torch.cuda.synchronize(dev)

    cfg = QuantConfig(**cfg_kwargs)
    heads, seq = args.heads, args.seq
    # weak scaling: rank r holds batch element r of a global batch of `world`
    maker = make_video_inputs if args.workload.startswith("wan14b_video") else make_inputs
    q, k, v = maker(batch, heads, seq, D_HEAD, 1234 + rank, dev)
    qp, kp, vp, pad = pad_like_hook(q, k, v, cfg)
    del q, k, v
    flops_per_step = 4.0 * batch * heads * seq * seq * D_HEAD          # unpadded, per GPU
    if seq_k is not None:
        # queries padded as above; the text keys / values have their own (block-aligned) length
        _, kp, vp = make_inputs(batch, heads, seq_k, D_HEAD, 4321 + rank, dev)
        flops_per_step = 4.0 * batch * heads * seq * seq_k * D_HEAD
        args.no_e2e = True                                              # the host-buffer entry takes equal shapes
        args.no_cpu_baseline = True
        args.no_verify = True
    lib = L.lib()

    brick_order = None
    if args.brick is not None:
        if not args.workload.startswith("wan14b_video"):
            raise SystemExit("--brick applies to the video workload (tokens on a (t, h, w) grid)")
        from low_bit_fake_quant.hook import fake_quant_attention_reordered, space_time_block_order
        bt, bh_, bw = (int(x) for x in args.brick.split(","))
        gt, gh, gw = VIDEO_GRID
        args.no_e2e = True                                              # the host-buffer entry has no reorder
        brick_order = space_time_block_order(gt, gh, gw, ts=bt, hs=bh_, ws=bw, tail=qp.shape[1] - gt * gh * gw, device=dev)

    def step(qq, kk, vv, c=cfg):
        if brick_order is not None:
            return fake_quant_attention_reordered(qq, kk, vv, c, brick_order,
                                                  _blasst_tile_predicate=args.blasst_tile_predicate)[:, :seq]
        if seq_k is not None:
            from low_bit_fake_quant.hook import fake_quant_cross_attention
            return fake_quant_cross_attention(qq, kk, vv, c)[:, :seq]
        o = fq.fake_quant_attention(qq, kk, vv, c, _reference_operands=args.reference_operands,
                                    _blasst_tile_predicate=args.blasst_tile_predicate and c.blasst_lambda is not None)
        return o[:, :seq]

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def timed(fn, steps, warmup):
        """`warmup` untimed and `steps` timed calls of fn, bracketed by barriers; returns (max-over-ranks ms per step,
        per-launch ms of the attention kernel, library launches per step)."""
        for _ in range(warmup):
            fn()
        barrier()
        K12.raise_if_device_error(dev)
        K12.KERNEL_EVENTS = []
        launches0 = lib.lbfq_launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        ms_total = ev0.elapsed_time(ev1)
        launches = int(lib.lbfq_launch_count() - launches0)
        kernel_ms = [a.elapsed_time(b) for a, b in K12.KERNEL_EVENTS]
        K12.KERNEL_EVENTS = None
        K12.raise_if_device_error(dev)
        t = torch.tensor([ms_total], device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps, (sum(kernel_ms) / max(len(kernel_ms), 1)), launches // max(steps, 1)

    # the clock sampler (an nvidia-smi child) is started before the warm-up: its start-up takes the driver's
    # locks for a few hundred ms, which would otherwise stall kernel launches inside a short timed region
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step(qp, kp, vp)
    barrier()
    if rank == 0:
        sampler.lines.clear()                      # keep only the samples taken during the timed regions

    # ---- timed region: inputs resident in HBM --------------------------------
    ms_step, k_ms, launches = timed(lambda: step(qp, kp, vp), args.steps, 0)
    fast = lib.lbfq_attention_last_variant() == 1
    value = world * flops_per_step / (ms_step * 1e-3) / 1e12

    # ---- the second stack of the same shape, same tensors (config.also) -------
    also = None
    if not args.no_also and args.workload in ALSO and seq_k is None and brick_order is None:
        a_name = ALSO[args.workload]
        a_cfg = QuantConfig(**WORKLOADS[a_name][0])
        if pad_like_hook(qp[:, :seq], kp[:, :seq], vp[:, :seq], a_cfg)[3] == pad:      # same padded length
            a_ms, a_kms, a_launches = timed(lambda: step(qp, kp, vp, a_cfg), args.steps, args.warmup)
            also = {"workload": a_name, "value": world * flops_per_step / (a_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": a_ms, "kernel_ms": a_kms, "gpu_launches_per_step": a_launches,
                    "roofline_frac": None}
    clocks = sampler.stop() if rank == 0 else None

    # ---- strong scaling: ONE problem (batch element 0) over the ranks, 40/N heads each --------------
    strong = None
    if world > 1 and not args.no_strong and seq_k is None and brick_order is None:
        lo, hi = slab_range(heads, world, rank)
        sq, sk, sv = (t[:, :, lo:hi].contiguous() for t in maker(batch, heads, seq, D_HEAD, 1234, dev))   # element 0 everywhere
        sq, sk, sv, _ = pad_like_hook(sq, sk, sv, cfg)

        def strong_step():
            o, _ = attention_on_shard(sq, sk, sv, cfg, world=world, rank=rank, sliced=True, total_heads=heads,
                                      _reference_operands=args.reference_operands)
            return o

        s_ms, _, _ = timed(strong_step, args.steps, args.warmup)
        strong = {"value": flops_per_step / (s_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": s_ms,
                  "heads_per_gpu": [b_ - a_ for a_, b_ in (slab_range(heads, world, r) for r in range(world))],
                  "note": "one 40-head problem partitioned over the ranks (sharding.attention_on_shard), no collective"}
        del sq, sk, sv

    # ---- end to end: pinned host buffers in, result back ----------------------
    e2e = None
    if not args.no_e2e:
        # the public host-buffer entry: heads chunks pipelined over copy-in / compute / copy-out streams
        hq, hk, hv = (x.cpu().pin_memory() for x in (qp, kp, vp))
        hout = torch.empty((batch, seq, heads, D_HEAD), dtype=qp.dtype).pin_memory()

        def e2e_step():
            fq.fake_quant_attention_host(hq, hk, hv, cfg, out=hout, device=dev, heads_per_chunk=args.e2e_heads_per_chunk,
                                         chunk_heads=e2e_chunks)

        e2e_chunks = [int(x) for x in args.e2e_chunks.split(",")] if args.e2e_chunks else None
        n_e2e = max(3, args.steps)
        ms_e2e, _, _ = timed(e2e_step, n_e2e, 2)

        # what the host's memory and links allow for these bytes: plain contiguous copies, all ranks at once
        def copy_only():
            qp.copy_(hq, non_blocking=True); kp.copy_(hk, non_blocking=True); vp.copy_(hv, non_blocking=True)
            hout.copy_(qp[:, :seq], non_blocking=True)

        ms_copy, _, _ = timed(copy_only, 3, 1)
        h2d = int(3 * hq.numel() * hq.element_size())
        d2h = int(hout.numel() * hout.element_size())
        e2e = {"value": world * flops_per_step / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "steps": n_e2e,
               "copy_ceiling": {"ms_per_step": ms_copy, "gb_per_s_per_gpu": (h2d + d2h) / (ms_copy * 1e-3) / 1e9,
                                "note": "the same bytes as plain copies from / to pinned memory, every rank at once, no compute: "
                                        "the lower bound of an unpipelined host-buffer step is this plus the device time"}}
        del hq, hk, hv

    parity = None
    if rank == 0 and not args.no_verify and brick_order is None and world == 1:
        parity = verify_one_head(qp, kp, vp, cfg, reference_operands=args.reference_operands)

    if rank == 0:
        bf16_peak, hbm_peak, peak_src = load_peaks()
        fp8_peak = 2.0 * bf16_peak          # dense FP8 tensor rate = 2 x the measured dense BF16 rate
        achieved = flops_per_step / (k_ms * 1e-3) / 1e12 if k_ms > 0 else 0.0
        kernel_name = "attn_fast_kernel<128,64>" if fast else "attn_kernel<128,64>"
        # DRAM bytes of one attention launch: ncu captures of 4-head launches of the same S, scaled by heads
        ent = load_traffic_table().get(f"{args.workload}:{'fast' if fast else 'general'}")
        traffic = ent["bytes_per_4_heads"] * heads / 4.0 if (ent and seq == S_REAL) else None
        roofline = {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
                    "frac": achieved / fp8_peak, "traffic": traffic, "kernel": kernel_name,
                    "kernel_ms": k_ms, "peak_source": f"2 x bf16_tflops ({peak_src})",
                    "step_frac": (flops_per_step / (ms_step * 1e-3) / 1e12) / fp8_peak}
        if also is not None:
            also["roofline_frac"] = (flops_per_step / (also["kernel_ms"] * 1e-3) / 1e12) / fp8_peak if also["kernel_ms"] > 0 else None
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            torch.set_num_threads(os.cpu_count() or 1)
            reps = 8 if cfg.q_kmeans_k is None else 4                  # about 10-30 s of host work
            tf, dt = cpu_oracle_sample(cfg_kwargs, seq=32768, heads=1, steps=reps)
            cpu = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": f"1 head x S=32768 of the workload (1/40 of a step) x {reps} repeats, {dt:.2f} s each, "
                             "oracle port on the host cores"}
        blasst = None
        if cfg.blasst_lambda is not None and cfg.smoothing != "full" and cfg.q_kmeans_k is None and cfg.v_kmeans_k is None:
            sq, sk_, sv = (qp, kp, vp) if brick_order is None else (x[:, brick_order].contiguous() for x in (qp, kp, vp))
            blasst = dict(blasst_skip_ratios(sq, sk_, sv, cfg, args.blasst_tile_predicate), blasst_lambda=cfg.blasst_lambda, blasst_fill=cfg.blasst_fill)
            if args.brick is not None:
                blasst["brick"] = args.brick
            if args.blasst_sweep and world == 1:
                grid = []
                for lam in (1e-4, 1e-3, 1e-2):
                    for fill in ("zero", "mean_a1.5", "uta16_a1.5"):
                        c2 = QuantConfig(**{**cfg_kwargs, "blasst_lambda": lam, "blasst_fill": fill})
                        g_ms, g_kms, _ = timed(lambda: step(qp, kp, vp, c2), max(3, args.steps // 2), 2)
                        r = blasst_skip_ratios(sq, sk_, sv, c2, args.blasst_tile_predicate)
                        grid.append({"blasst_lambda": lam, "blasst_fill": fill, "ms_per_step": g_ms, "kernel_ms": g_kms,
                                     "row_skip_ratio": r["row_skip_ratio"], "tile_skip_ratio": r["tile_skip_ratio"]})
                blasst["sweep"] = grid
        p_note = {"dynamic": "P re-scaled per (row, block) and handed to a BF16 P.V as the reference rounds it",
                  "elementwise": "P as e4m3 codes, FP8 P.V"}.get(cfg.p_quant, "P per the V kind")
        line = {
            "metric": "fused FP8 fake-quant attn TFLOP/s at 40x32760x128", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 (reference-operand mode)" if args.reference_operands else f"fp8_e4m3 Q.K^T; {p_note}", "data": "synthetic",
            "config": {"workload": args.workload + ("+reference_operands" if args.reference_operands else ""), "B_per_gpu": batch, "global_batch": batch * world, "H": heads,
                       "S": seq, "S_padded": seq + pad, "S_keys": seq_k if seq_k is not None else seq, "D": D_HEAD, "input_dtype": "bf16",
                       "l2": "inputs (3 x %.0f MB) exceed the 126 MB L2" % (qp.numel() * 2 / 1e6),
                       "parallelism": f"batch x heads sharded over {world} GPU(s), no collective", "also": also},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches * args.steps,
            "gpu_launches_per_step": launches, "clocks": clocks, "parity": parity, "strong_scaling": strong,
        }
        if blasst is not None:
            line["config"]["blasst"] = blasst       # flops are not reduced for skipped row-blocks
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
