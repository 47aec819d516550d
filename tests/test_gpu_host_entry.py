"""The host-buffer entry pipelines heads chunks over three streams; its result must be bit-identical to one
device-resident call on the whole tensors (every (batch, head) slab is independent; Hadamard signs and k-means
seeding are indexed by the global head)."""
import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant.attention_triton import raise_if_device_error
from low_bit_fake_quant.config import QuantConfig

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CFGS = {
    "k_smooth_static": dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64, smoothing="k_only",
                            q_kmeans_k=None),
    "full_dynamic_kmeans_hadamard": dict(qk_quant="fp8_block", v_quant="fp8_channel", fp8_block_size=64,
                                         q_smooth_block_size=64, smoothing="full", q_kmeans_k=8, v_kmeans_k=8,
                                         v_smooth_mode="per_block", p_quant="dynamic", rowmax_mode="qm_k",
                                         qk_hadamard=True),
    "mxfp8": dict(qk_quant="mxfp8", v_quant="mxfp8", smoothing="off", q_kmeans_k=None, qk_hadamard=True),
}


@pytest.mark.parametrize("name", sorted(CFGS))
@pytest.mark.parametrize("pinned", [True, False])
def test_host_entry_equals_device_entry(name, pinned):
    cfg = QuantConfig(**CFGS[name])
    torch.manual_seed(11)
    B, S, H, D = 2, 512, 5, 128
    q, k, v = (torch.randn(B, S, H, D).bfloat16() for _ in range(3))
    if pinned:
        q, k, v = q.pin_memory(), k.pin_memory(), v.pin_memory()
    want = fq.fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg).cpu()
    got = fq.fake_quant_attention_host(q, k, v, cfg, heads_per_chunk=2)           # chunks of 2, 2, 1 heads
    raise_if_device_error(torch.device(DEV))
    assert got.shape == q.shape and got.dtype == q.dtype and not got.is_cuda
    assert torch.equal(got, want)


def test_host_entry_brings_back_only_the_rows_asked_for():
    cfg = QuantConfig(**CFGS["k_smooth_static"])
    torch.manual_seed(12)
    q, k, v = (torch.randn(1, 512, 3, 64).bfloat16().pin_memory() for _ in range(3))
    want = fq.fake_quant_attention(q.to(DEV), k.to(DEV), v.to(DEV), cfg).cpu()
    out = torch.full((1, 500, 3, 64), 7.0, dtype=torch.bfloat16).pin_memory()
    got = fq.fake_quant_attention_host(q, k, v, cfg, out=out, heads_per_chunk=1)
    assert got is out and torch.equal(out, want[:, :500])


def test_host_entry_errors():
    x = torch.zeros(1, 128, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="host memory"):
        fq.fake_quant_attention_host(x.to(DEV), x, x)
    with pytest.raises(ValueError, match="shapes must match"):
        fq.fake_quant_attention_host(x, x[:, :64], x)
    with pytest.raises(ValueError, match="out must be"):
        fq.fake_quant_attention_host(x, x, x, out=torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        fq.fake_quant_attention_host(x.double(), x.double(), x.double())
