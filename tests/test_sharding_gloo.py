"""The multi-GPU layout of the path, exercised as two gloo ranks on CPU.

Each rank owns a contiguous range of heads (``sharding.slab_range``), runs the
path on its shard alone -- here through the CPU oracle, told where the shard
sits in the full problem -- and the concatenation must equal the unsharded
run bit for bit. No collective is used on the data path; ``all_gather`` only
assembles the result for the comparison, and ``all_reduce(MAX)`` is the
max-over-ranks timing rule of the benchmark.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from low_bit_fake_quant.config import QuantConfig
from low_bit_fake_quant.sharding import head_shard, slab_range
from oracle import api as OA

CFG = dict(fp8_block_size=64, q_smooth_block_size=64, smoothing="full", q_kmeans_k=4, v_kmeans_k=4,
           v_smooth_mode="per_block", p_quant="dynamic", rowmax_mode="qm_k", qk_hadamard=True)


def _inputs():
    g = torch.Generator().manual_seed(42)
    return tuple(torch.randn(1, 128, 4, 64, generator=g).bfloat16() for _ in range(3))


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        q, k, v = _inputs()
        cfg = QuantConfig(**CFG)
        qs, ks, vs, off = head_shard(q, k, v, world, rank)
        assert (off, off + qs.shape[2]) == slab_range(4, world, rank)
        out = OA.fake_quant_attention(qs, ks, vs, cfg, faithful=False, head_offset=off, total_heads=4)
        parts = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(parts, out)                       # assembly for the check only
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)          # timing rule: max over ranks
        if rank == 0:
            ret["out"] = torch.cat(parts, dim=2)
            ret["tmax"] = t.item()
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharding_equals_unsharded():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    q, k, v = _inputs()
    full = OA.fake_quant_attention(q, k, v, QuantConfig(**CFG), faithful=False)
    assert ret["tmax"] == 2.0
    assert torch.equal(ret["out"], full)
