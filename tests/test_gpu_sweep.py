"""Randomised sweep of configurations against the oracle.

The hand-written cases of the other files each pin one feature; this one draws whole configurations (quantizer kinds,
smoothing, k-means, rotation, P modes, BLASST fills, block sizes, ragged lengths, input dtypes, softmax scales) from a
seeded generator and holds every draw to the path's parity bound. It found three combinations that the hand-written
cases had missed (V-scale blocks that are not the smoothing blocks; smoothing blocks that do not tile a 128-key stage;
the row-max estimate for inputs that are not BF16)."""
import random

import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant import _lib as L
from low_bit_fake_quant.attention import _preprocess
from low_bit_fake_quant.attention_triton import raise_if_device_error
from low_bit_fake_quant.config import QuantConfig
from oracle import api as OA

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FILLS = ["zero", "mean_a1.5", "uta16_a1.5", "uta8", "uta4_a0.5", "uta2", "max_a0.25", "logn", "sample8_a1.25", "thr_a0.25"]


def _draw(rnd):
    bn = rnd.choice([32, 64])
    kw = dict(qk_quant=rnd.choice(["fp8_block", "fp8_block", "mxfp8"]),
              v_quant=rnd.choice(["fp8_channel", "fp8_channel", "fp8_block", "mxfp8"]),
              fp8_block_size=rnd.choice([64, 64, 128]), smoothing=rnd.choice(["off", "k_only", "full"]),
              q_smooth_block_size=rnd.choice([64, 128, 192, 256]), q_kmeans_k=rnd.choice([None, None, 4]),
              v_kmeans_k=rnd.choice([None, None, 4]), v_smooth_mode=rnd.choice(["off", "per_block"]),
              v_smooth_block_size=rnd.choice([64, 64, 128, 192]), p_max_offset=rnd.choice([8, 8, 0, 4]),
              p_quant=rnd.choice(["auto", "elementwise", "dynamic", "mx"]), rowmax_mode="online",
              qk_hadamard=rnd.choice([False, False, True]), p_requant_block_m=bn, p_requant_block_n=bn,
              v_fp8_block_size=rnd.choice([64, 64, 128]), v_mxfp8_block_size=64)
    if kw["smoothing"] == "full" and rnd.random() < 0.5:
        kw["rowmax_mode"] = "qm_k"
    if rnd.random() < 0.3:
        kw["blasst_lambda"] = rnd.choice([1e-1, 1e-2])
        kw["blasst_fill"] = rnd.choice(FILLS)
    if kw["p_quant"] == "mx":
        kw["p_mx_block_n"] = bn
    shape = dict(B=rnd.choice([1, 2]), H=rnd.choice([1, 2, 3]), D=rnd.choice([64, 128]),
                 S=rnd.choice([64, 192, 256, 320, 448, 576, 704, 768, 1024, 1344]),
                 dtype=rnd.choice([torch.bfloat16, torch.bfloat16, torch.float16, torch.float32]),
                 sm_scale=rnd.choice([None, None, 0.05, 0.2]))
    return kw, shape


@pytest.mark.parametrize("seed", [1, 2, 11, 12, 13])
def test_random_configurations_match_the_oracle(seed):
    rnd = random.Random(seed)
    ran = 0
    for it in range(60):
        kw, sh = _draw(rnd)
        S = sh["S"]
        if any(S % kw[n] for n in ("q_smooth_block_size", "fp8_block_size", "v_smooth_block_size", "v_fp8_block_size")):
            continue
        cfg = QuantConfig(**kw)
        torch.manual_seed(1000 * seed + it)
        q = torch.randn(sh["B"], S, sh["H"], sh["D"])
        k = torch.randn(sh["B"], S, sh["H"], sh["D"]) + 2 * torch.randn(1, 1, sh["H"], sh["D"])
        v = torch.randn(sh["B"], S, sh["H"], sh["D"])
        q[..., :4] *= 4
        k[..., :4] *= 4
        q, k, v = (t.to(sh["dtype"]) for t in (q, k, v))
        try:
            g = fq.fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg, sm_scale=sh["sm_scale"], _debug_fp32=True)
        except (ValueError, NotImplementedError):
            continue                                        # a combination the path refuses (with a message)
        raise_if_device_error(torch.device(DEV))
        g = g.float().cpu()
        fast = L.lib().lbfq_attention_last_variant() == 1
        ql = vl = None
        if cfg.q_kmeans_k is not None or cfg.v_kmeans_k is not None:   # k-means labels are not pinned: hand over the GPU's
            pre = _preprocess(q.to(DEV), k.to(DEV), v.to(DEV), cfg)
            ql = pre[5].labels.cpu() if pre[5] is not None else None
            vl = pre[6].labels.cpu() if pre[6] is not None else None
        o = OA.fake_quant_attention(q, k, v, cfg, sm_scale=sh["sm_scale"], faithful=False, out_fp32=True,
                                    q_labels=ql, v_labels=vl, p_bf16=fast)
        rep = OA.parity_report(g, o, q, k, v, sm_scale=sh["sm_scale"])
        assert torch.isfinite(g).all() and OA.parity_ok(rep), (it, fast, sh, kw, rep)
        ran += 1
    assert ran >= 8


@pytest.mark.parametrize("seed", [5, 54])
def test_random_configurations_host_entry_equals_device_entry(seed):
    """The host-buffer entry (heads chunks pipelined over three streams) against one device-resident call, bit for
    bit, over drawn configurations, head counts and chunk sizes."""
    rnd = random.Random(seed)
    ran = 0
    for it in range(60):
        kw, sh = _draw(rnd)
        S = sh["S"]
        if any(S % kw[n] for n in ("q_smooth_block_size", "fp8_block_size", "v_smooth_block_size", "v_fp8_block_size")):
            continue
        heads, chunk = rnd.choice([3, 5, 6]), rnd.choice([1, 2, 4])
        cfg = QuantConfig(**kw)
        torch.manual_seed(1000 * seed + it)
        q, k, v = (torch.randn(sh["B"], S, heads, sh["D"]).to(sh["dtype"]) for _ in range(3))
        k = k + 1
        try:
            want = fq.fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg, sm_scale=sh["sm_scale"]).cpu()
        except (ValueError, NotImplementedError):
            continue
        got = fq.fake_quant_attention_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), cfg, sm_scale=sh["sm_scale"],
                                           heads_per_chunk=chunk)
        raise_if_device_error(torch.device(DEV))
        assert torch.equal(got, want), (it, heads, chunk, sh, kw)
        ran += 1
    assert ran >= 8
