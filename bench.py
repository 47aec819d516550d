#!/usr/bin/env python
"""Benchmark of the fake-quant attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one call of ``low_bit_fake_quant.fake_quant_attention`` on the
Wan-14B self-attention shape (B=1, H=40, S=32760 padded to 32768 by the
reference hook's rule, D=128, BF16) with the ``k_smooth_static`` stack
(fp8_block 64 Q/K, fp8_channel V, K smoothing, elementwise P*256, online row
max, 64x64 blocks) -- quantizers and the attention kernel together. With N > 1
(launched under torchrun) every rank runs one such problem on its own GPU: the
path has no collective, so scaling is weak (global batch = N).

Printed JSON (rank 0): throughput in TFLOP/s with the algorithmic flop count
4*B*H*Sq*Sk*D on the unpadded shape; ``e2e`` is the same call fed from pinned
host buffers with the result copied back; ``roofline`` describes the
attention kernel against the dense-FP8 tensor peak; ``cpu_baseline`` is the
CPU restatement of the reference timed on a bounded sample.
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


def blasst_skip_ratios(qp, kp, vp, cfg):
    """Row-skip and whole-program skip ratios from the kernel's stats tensor, computed the way the reference's BLASST
    evaluation does (bench/eval_blasst_quant.py:216-227). One extra call, outside the timed region."""
    import low_bit_fake_quant as fq
    from low_bit_fake_quant.attention import _fake_quant_attention_p_requant
    k_work = fq.smooth_k(kp)[0] if cfg.smoothing != "off" else kp
    _, stats = _fake_quant_attention_p_requant(qp, k_work, vp, None, None, None, cfg, 1.0 / math.sqrt(qp.shape[-1]),
                                               qp.dtype, return_stats=True)
    skipped, total = float(stats[..., 0].sum().item()), float(stats[..., 1].sum().item())
    tiles = stats[..., 1].gt(0)
    tile_skipped = float((stats[..., 0] == stats[..., 1]).logical_and(tiles).sum().item())
    return {"row_skip_ratio": skipped / total if total > 0 else 0.0,
            "tile_skip_ratio": tile_skipped / float(tiles.sum().item()) if tiles.any() else 0.0,
            "skipped_row_blocks": skipped, "total_row_blocks": total}


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
    seq, heads = 16384, 1
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
    ap.add_argument("--workload", default="wan14b_self_attn_k_smooth_static", choices=sorted(WORKLOADS))
    ap.add_argument("--heads", type=int, default=H_FULL, help="heads per GPU (smaller values are for profiling runs only)")
    ap.add_argument("--seq", type=int, default=S_REAL)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-heads-per-chunk", type=int, default=None,
                    help="heads per pipelined chunk of the host-buffer entry (default: the entry's own choice)")
    ap.add_argument("--reference-operands", action="store_true",
                    help="run path B on the reference's own BF16 operands (BF16 MMAs) instead of the FP8 codes; not the headline")
    ap.add_argument("--blasst-lambda", type=float, default=None, help="override the BLASST threshold of a BLASST workload")
    ap.add_argument("--blasst-fill", default=None, help="override the BLASST fill of a BLASST workload (zero, mean_a1.5, uta16_a1.5 ...)")
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

    def step(qq, kk, vv):
        if brick_order is not None:
            return fake_quant_attention_reordered(qq, kk, vv, cfg, brick_order)[:, :seq]
        if seq_k is not None:
            from low_bit_fake_quant.hook import fake_quant_cross_attention
            return fake_quant_cross_attention(qq, kk, vv, cfg)[:, :seq]
        o = fq.fake_quant_attention(qq, kk, vv, cfg, _reference_operands=args.reference_operands)
        return o[:, :seq]

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # the clock sampler (an nvidia-smi child) is started before the warm-up: its start-up takes the driver's
    # locks for a few hundred ms, which would otherwise stall kernel launches inside a short timed region
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        out = step(qp, kp, vp)
    barrier()
    K12.raise_if_device_error(dev)
    if rank == 0:
        sampler.lines.clear()                      # keep only the samples taken during the timed region

    # ---- timed region: inputs resident in HBM --------------------------------
    K12.KERNEL_EVENTS = []
    launches0 = lib.lbfq_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        out = step(qp, kp, vp)
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = int(lib.lbfq_launch_count() - launches0)
    kernel_ms = [a.elapsed_time(b) for a, b in K12.KERNEL_EVENTS]
    K12.KERNEL_EVENTS = None
    clocks = sampler.stop() if rank == 0 else None
    K12.raise_if_device_error(dev)
    t = torch.tensor([ms_total], device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = world * flops_per_step / (ms_step * 1e-3) / 1e12

    # ---- end to end: pinned host buffers in, result back ----------------------
    e2e = None
    if not args.no_e2e:
        # the public host-buffer entry: heads chunks pipelined over copy-in / compute / copy-out streams
        hq, hk, hv = (x.cpu().pin_memory() for x in (qp, kp, vp))
        hout = torch.empty((batch, seq, heads, D_HEAD), dtype=qp.dtype).pin_memory()

        def e2e_step():
            fq.fake_quant_attention_host(hq, hk, hv, cfg, out=hout, device=dev, heads_per_chunk=args.e2e_heads_per_chunk)

        for _ in range(2):
            e2e_step()
        barrier()
        n_e2e = max(2, min(args.steps, 5))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e2e = float(te.item()) / n_e2e
        e2e = {"value": world * flops_per_step / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(3 * hq.numel() * hq.element_size()),
               "d2h_bytes_per_step": int(hout.numel() * hout.element_size()), "ms_per_step": ms_e2e}
        del hq, hk, hv

    if rank == 0:
        bf16_peak, hbm_peak, peak_src = load_peaks()
        fp8_peak = 2.0 * bf16_peak          # dense FP8 tensor rate = 2 x the measured dense BF16 rate
        k_ms = sum(kernel_ms) / max(len(kernel_ms), 1)
        achieved = flops_per_step / (k_ms * 1e-3) / 1e12 if k_ms > 0 else 0.0
        # DRAM bytes of one attention launch, measured by ncu on a 4-head launch of the same S and scaled by heads
        # (each head's traffic is independent): 55.5 MB for the TMEM-resident kernel on the k_smooth_static stack, 171.1 MB
        # on the full_dynamic stack (profiles/attn_fast_kernel_wan14b_*.md), 136.6 MB for the general kernel on the
        # full_dynamic stack (profiles/attn_kernel_wan14b_full_dynamic.md)
        fast = lib.lbfq_attention_last_variant() == 1
        traffic = None
        if seq == S_REAL and fast and args.workload == "wan14b_self_attn_k_smooth_static":
            traffic = 55.47e6 * heads / 4.0
        elif seq == S_REAL and args.workload == "wan14b_self_attn_full_dynamic":
            traffic = (171.1e6 if fast else 136.6e6) * heads / 4.0
        roofline = {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
                    "frac": achieved / fp8_peak, "traffic": traffic, "kernel": "attn_fast_kernel<128,64>" if lib.lbfq_attention_last_variant() == 1 else "attn_kernel<128,64>",
                    "kernel_ms": k_ms, "peak_source": f"2 x bf16_tflops ({peak_src})"}
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            torch.set_num_threads(os.cpu_count() or 1)
            reps = 8                                   # about 10-20 s of host work
            tf, dt = cpu_oracle_sample(cfg_kwargs, seq=32768, heads=1, steps=reps)
            cpu = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": f"1 head x S=32768 of the workload (1/40 of a step) x {reps} repeats, {dt:.2f} s each, "
                             "oracle port on the host cores"}
        blasst = None
        if cfg.blasst_lambda is not None and cfg.smoothing != "full" and cfg.q_kmeans_k is None and cfg.v_kmeans_k is None:
            sq, sk_, sv = (qp, kp, vp) if brick_order is None else (x[:, brick_order].contiguous() for x in (qp, kp, vp))
            blasst = dict(blasst_skip_ratios(sq, sk_, sv, cfg), blasst_lambda=cfg.blasst_lambda, blasst_fill=cfg.blasst_fill)
            if args.brick is not None:
                blasst["brick"] = args.brick
        line = {
            "metric": "fused FP8 fake-quant attn TFLOP/s at 40x32760x128", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 (reference-operand mode)" if args.reference_operands else "fp8_e4m3", "data": "synthetic",
            "config": {"workload": args.workload + ("+reference_operands" if args.reference_operands else ""), "B_per_gpu": batch, "global_batch": batch * world, "H": heads,
                       "S": seq, "S_padded": seq + pad, "S_keys": seq_k if seq_k is not None else seq, "D": D_HEAD, "input_dtype": "bf16",
                       "l2": "inputs (3 x %.0f MB) exceed the 126 MB L2" % (qp.numel() * 2 / 1e6),
                       "parallelism": f"batch x heads sharded over {world} GPU(s), no collective"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        }
        if blasst is not None:
            line["config"]["blasst"] = blasst       # flops are not reduced for skipped row-blocks
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
