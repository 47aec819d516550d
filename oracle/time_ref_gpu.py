"""Times the reference's own Triton path on the GPU this runs on, at the benchmark shape.

TEST / MEASUREMENT INFRASTRUCTURE ONLY (nothing in the package imports it). Needs the reference package staged under
``oracle/_ref`` (``oracle/make_ref.py``) and Triton. The reference's k-means dependency (``flash_kmeans``) is not
installed here, so its cluster labels are injected (``oracle/ref_gpu.py``): the reference's time below therefore
EXCLUDES its k-means, while the library's time next to it includes its own.

    python oracle/time_ref_gpu.py [workload ...]      # workloads of bench.py; default: the two benchmark stacks
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "low-bit-attention-fake-quant_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import bench                                             # noqa: E402
import low_bit_fake_quant as fq                          # noqa: E402
from low_bit_fake_quant.config import QuantConfig        # noqa: E402
from oracle import ref_gpu as RG                         # noqa: E402


def timed(fn, steps=3, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def main():
    ref = RG.load()
    if ref is None:
        print(json.dumps({"unavailable": "the reference package is not staged under oracle/_ref, or Triton is missing"}))
        return
    dev = torch.device("cuda:0")
    names = sys.argv[1:] or ["wan14b_self_attn_k_smooth_static", "wan14b_self_attn_full_dynamic"]
    for name in names:
        cfg_kwargs, batch = bench.WORKLOADS[name][:2]
        cfg = QuantConfig(**cfg_kwargs)
        q, k, v = bench.make_inputs(batch, bench.H_FULL, bench.S_REAL, bench.D_HEAD, 1234, dev)
        qp, kp, vp, _ = bench.pad_like_hook(q, k, v, cfg)
        del q, k, v
        labels = []
        if cfg.q_kmeans_k is not None or cfg.v_kmeans_k is not None:
            pc = fq.prepare_for_attention(qp, kp, vp, cfg)
            labels = [t.labels.to(torch.int32) for t in (pc.q_kmeans, pc.v_kmeans) if t is not None]
            del pc
        rcfg = ref.QuantConfig(**cfg_kwargs)

        def ref_step():
            RG.inject_labels(*labels)
            return ref.fake_quant_attention(qp, kp, vp, rcfg)

        ours_ms = timed(lambda: fq.fake_quant_attention(qp, kp, vp, cfg))
        ref_ms = timed(ref_step)
        cos = torch.nn.functional.cosine_similarity(ref_step().float().flatten(), fq.fake_quant_attention(qp, kp, vp, cfg).float().flatten(), dim=0)
        flops = 4.0 * batch * bench.H_FULL * bench.S_REAL * bench.S_REAL * bench.D_HEAD
        print(json.dumps({"workload": name, "reference_triton_ms": ref_ms, "library_ms": ours_ms, "ratio": ref_ms / ours_ms,
                          "reference_tflops": flops / ref_ms / 1e9, "library_tflops": flops / ours_ms / 1e9,
                          "cosine_between_outputs": float(cos), "triton": __import__("triton").__version__,
                          "note": "reference time excludes its k-means (labels injected); the library's includes its own"}))
        del qp, kp, vp


if __name__ == "__main__":
    main()
