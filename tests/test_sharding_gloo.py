"""The multi-GPU layout of the path, exercised as gloo ranks on CPU.

Each rank calls the package's own ``sharding.attention_on_shard`` -- the call ``bench.py`` makes on a GPU rank --
which slices the rank's contiguous range of heads, tells the attention entry where the shard sits in the full
problem and returns the local result; ``sharding.gather_heads`` assembles the full output. The attention entry
itself needs a GPU, so the CPU oracle stands in for it here (same two keywords): what this covers is the host
logic of the N > 1 path -- ranges, offsets, uneven shards, the gather -- and that a sharded run equals the
unsharded one bit for bit. No collective is used on the data path; ``all_reduce(MAX)`` is the max-over-ranks
timing rule of the benchmark.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from low_bit_fake_quant.config import QuantConfig
from low_bit_fake_quant.sharding import attention_on_shard, gather_heads, slab_range
from oracle import api as OA

CFG = dict(fp8_block_size=64, q_smooth_block_size=64, smoothing="full", q_kmeans_k=4, v_kmeans_k=4,
           v_smooth_mode="per_block", p_quant="dynamic", rowmax_mode="qm_k", qk_hadamard=True)


HEADS = 5          # not divisible by the world sizes below: uneven shards


def _inputs():
    g = torch.Generator().manual_seed(42)
    return tuple(torch.randn(1, 128, HEADS, 64, generator=g).bfloat16() for _ in range(3))


def _oracle_as_attention(q, k, v, cfg, *, _head_offset, _total_heads):
    return OA.fake_quant_attention(q, k, v, cfg, faithful=False, head_offset=_head_offset, total_heads=_total_heads)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        q, k, v = _inputs()
        cfg = QuantConfig(**CFG)
        out, off = attention_on_shard(q, k, v, cfg, world=world, rank=rank, attention=_oracle_as_attention)
        assert (off, off + out.shape[2]) == slab_range(HEADS, world, rank)
        # the same call fed with the rank's own slice (how a rank that never holds the full tensors calls it)
        lo, hi = slab_range(HEADS, world, rank)
        out2, _ = attention_on_shard(q[:, :, lo:hi], k[:, :, lo:hi], v[:, :, lo:hi], cfg, world=world, rank=rank,
                                     attention=_oracle_as_attention, sliced=True, total_heads=HEADS)
        assert torch.equal(out, out2)
        full = gather_heads(out, HEADS)                   # assembly for the check only
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)          # timing rule: max over ranks
        if rank == 0:
            ret["out"] = full
            ret["tmax"] = t.item()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_head_sharding_equals_unsharded(world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    q, k, v = _inputs()
    full = OA.fake_quant_attention(q, k, v, QuantConfig(**CFG), faithful=False)
    assert ret["tmax"] == float(world)
    assert torch.equal(ret["out"], full)
