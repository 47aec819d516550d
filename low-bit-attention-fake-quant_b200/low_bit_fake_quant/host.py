"""Host-buffer entry: ``fake_quant_attention`` for callers whose Q, K, V live in host memory.

The reference has no such entry (its callers hold CUDA tensors,
src/low_bit_fake_quant/attention.py:741-742). Every (batch, head) slab of the
operator is independent end to end (the k-means rows, the K mean, every scale
tensor and the attention grid are all indexed by head), so the heads are cut
into chunks and pipelined over three streams: while chunk ``i`` is computed,
chunk ``i + 1`` travels host -> device and the result of chunk ``i - 1`` travels
device -> host. The result is bit-identical to one call on the whole tensors:
Hadamard signs and k-means seeding are indexed by the global head.
"""
from __future__ import annotations

import time
from typing import Optional, Sequence

import torch

from . import _lib as L
from .attention import fake_quant_attention
from .config import QuantConfig


def _copy_rows(dst: torch.Tensor, src: torch.Tensor, h0: int, h1: int, rows_s: int, to_device: bool, stream) -> None:
    """(B, :rows_s, h0:h1, D) of the host tensor <-> a contiguous (B, S_dev, h1-h0, D) device tensor."""
    host, dev = (src, dst) if to_device else (dst, src)
    b, s_host, h, d = host.shape
    es = host.element_size()
    width = (h1 - h0) * d * es
    for bi in range(b):
        hp = host.data_ptr() + (bi * s_host * h + h0) * d * es
        dp = dev.data_ptr() + bi * dev.shape[1] * width
        if to_device:
            L.check(L.lib().lbfq_copy_rows_async(dp, width, hp, h * d * es, width, rows_s, 1, stream.cuda_stream))
        else:
            L.check(L.lib().lbfq_copy_rows_async(hp, h * d * es, dp, width, width, rows_s, 0, stream.cuda_stream))


def _chunk_bounds(h: int, cfg: QuantConfig, heads_per_chunk: Optional[int], chunk_heads: Optional[Sequence[int]]):
    """[h0, h1) of every pipelined chunk of the H heads."""
    if chunk_heads is not None:
        sizes = [int(n) for n in chunk_heads]
        if not sizes or min(sizes) <= 0 or sum(sizes) != h:
            raise ValueError(f"chunk_heads must be positive and add up to the {h} heads; got {list(chunk_heads)}")
        edges = [0]
        for n in sizes:
            edges.append(edges[-1] + n)
        return list(zip(edges[:-1], edges[1:]))
    kmeans = cfg.q_kmeans_k is not None or cfg.v_kmeans_k is not None
    if heads_per_chunk is None:
        # small chunks hide more of the copies; the k-means passes want enough heads per launch to fill the GPU
        heads_per_chunk = 8 if kmeans else 4
    if heads_per_chunk <= 0:
        raise ValueError("heads_per_chunk must be positive")
    hc = min(heads_per_chunk, h)
    bounds = [(h0, min(h0 + hc, h)) for h0 in range(0, h, hc)]
    if len(bounds) > 2 and not kmeans:
        # nothing overlaps the last chunk's compute and copy back: taper it (.., hc/2, hc/4, .., 1) so that the tail
        # of the pipeline is one head long; the k-means passes keep their full chunks
        h0, h1 = bounds.pop()
        n = h1 - h0
        while n > 1:
            step = (n + 1) // 2
            bounds.append((h0, h0 + step))
            h0, n = h0 + step, n - step
        bounds.append((h0, h1))
    if len(bounds) > 2 and kmeans and hc >= 4:
        # nothing overlaps the first chunk's copy in: it is cut into a quarter and the rest, so that the kernels start
        # after a quarter of that copy (measured on the benchmark's full stack: 40.4 -> 39.1 ms per step)
        h0, h1 = bounds[0]
        cut = h0 + max(1, (h1 - h0) // 4)
        bounds[0:1] = [(h0, cut), (cut, h1)]
    return bounds


def fake_quant_attention_host(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cfg: Optional[QuantConfig] = None,
    *,
    sm_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    device: Optional[torch.device] = None,
    heads_per_chunk: Optional[int] = None,
    chunk_heads: Optional[Sequence[int]] = None,
    trace: Optional[list] = None,
) -> torch.Tensor:
    """``fake_quant_attention`` on host tensors.

    ``q, k, v``: contiguous (B, S, H, D) CPU tensors (pinned memory makes the copies asynchronous).
    ``out``: optional contiguous (B, S_out <= S, H, D) CPU tensor of ``q``'s dtype; only its first ``S_out``
    rows are brought back (the caller's way to drop padding rows). Returns ``out``; it is complete when
    this function returns. ``heads_per_chunk``: heads per pipelined chunk (default 4 with a tapered tail, or 8 with a
    k-means reorder, the first chunk then cut in two).
    ``chunk_heads``: the chunk sizes themselves, in order (they must add up to H); overrides ``heads_per_chunk``.
    ``trace``: a list that receives one record per chunk -- its heads and the device times (ms since the call's first
    copy was queued) at which its copy in, its kernels and its copy back ended, plus the host time its launches took.
    """
    if cfg is None:
        cfg = QuantConfig()
    if q.shape != k.shape or q.shape != v.shape:
        raise ValueError(f"q/k/v shapes must match; got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if q.ndim != 4:
        raise ValueError(f"q/k/v must be 4-D (B,S,H,D); got {q.shape}")
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("q/k/v must live in host memory; use fake_quant_attention for CUDA tensors")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q/k/v must share a dtype")
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError(f"unsupported dtype {q.dtype}")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("q/k/v must be contiguous")
    b, s, h, d = q.shape
    if out is None:
        out = torch.empty_like(q, pin_memory=q.is_pinned())
    if out.ndim != 4 or out.shape[0] != b or out.shape[2] != h or out.shape[3] != d or out.shape[1] > s:
        raise ValueError(f"out must be (B, S_out <= S, H, D); got {tuple(out.shape)}")
    if out.dtype != q.dtype or out.is_cuda or not out.is_contiguous():
        raise ValueError("out must be a contiguous host tensor of q's dtype")
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    bounds = _chunk_bounds(h, cfg, heads_per_chunk, chunk_heads)
    hc = max(h1 - h0 for h0, h1 in bounds)
    s_out = out.shape[1]

    with torch.cuda.device(dev):
        comp = torch.cuda.current_stream(dev)
        s_in, s_back = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        s_in.wait_stream(comp)
        slots = [[torch.empty((b, s, hc, d), dtype=q.dtype, device=dev) for _ in range(3)] for _ in range(2)]
        timing = trace is not None
        loaded = [torch.cuda.Event(enable_timing=timing) for _ in bounds]
        computed = [torch.cuda.Event(enable_timing=timing) for _ in bounds]
        returned = [torch.cuda.Event(enable_timing=True) for _ in bounds] if timing else None
        start = torch.cuda.Event(enable_timing=True) if timing else None
        host_ms = []
        results = []

        def buffers(i):
            n = bounds[i][1] - bounds[i][0]
            return [t[:, :, :n] if n == hc else t.view(-1)[: b * s * n * d].view(b, s, n, d) for t in slots[i % 2]]

        def load(i):
            h0, h1 = bounds[i]
            if i >= 2:
                s_in.wait_event(computed[i - 2])            # the slot's previous occupant has been consumed
            for dst, src in zip(buffers(i), (q, k, v)):
                _copy_rows(dst, src, h0, h1, s, True, s_in)
            loaded[i].record(s_in)

        if timing:
            start.record(s_in)
        load(0)
        for i, (h0, h1) in enumerate(bounds):
            if i + 1 < len(bounds):
                load(i + 1)                                  # queued before this chunk's launches: the host never holds it back
            bufs = buffers(i)
            comp.wait_event(loaded[i])
            t_host = time.perf_counter() if timing else 0.0
            o = fake_quant_attention(bufs[0], bufs[1], bufs[2], cfg, sm_scale=sm_scale, _head_offset=h0, _total_heads=h)
            if timing:
                host_ms.append((time.perf_counter() - t_host) * 1e3)
            computed[i].record(comp)
            s_back.wait_event(computed[i])
            o.record_stream(s_back)
            _copy_rows(out, o, h0, h1, s_out, False, s_back)
            if timing:
                returned[i].record(s_back)
            results.append(o)
        s_back.synchronize()
        comp.synchronize()
        L.status_for(dev)                 # everything has completed: raise if any launch gave up a bounded wait
        if timing:
            for i, (h0, h1) in enumerate(bounds):
                trace.append({"heads": h1 - h0, "copied_in_ms": start.elapsed_time(loaded[i]),
                              "computed_ms": start.elapsed_time(computed[i]), "copied_back_ms": start.elapsed_time(returned[i]),
                              "host_launch_ms": host_ms[i]})
    return out
