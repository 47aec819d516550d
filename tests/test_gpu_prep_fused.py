"""The fused preparation kernel against the chain of separate kernels it replaces: bit for bit.

``prepare.prep_fused`` gathers, smooths, rotates and quantises one tensor in a single pass; the separate functions of
the package (``kmeans._gather``, ``smooth_k`` / ``group_mean_q`` / ``smooth_v_per_block``, ``apply_qk_hadamard``, the
quantizers) are the statement of what it must return -- and they in turn are held to the oracle and to the recorded
reference vectors elsewhere. Also: ``fake_quant_attention`` with and without the fused path gives identical bits.
"""
import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant import _lib as L
from low_bit_fake_quant.attention_triton import raise_if_device_error
from low_bit_fake_quant.config import QuantConfig
from low_bit_fake_quant.kmeans import _gather
from low_bit_fake_quant.preprocess import k_channel_mean
from low_bit_fake_quant.prepare import group_rows, hadamard_signs, prep_fused

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _x(B, S, H, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, H, D, generator=g)
    x[..., 1] *= 8.0
    x = x + 1.5 * torch.randn(1, 1, H, D, generator=g) + 0.3 * torch.randn(B, S // 64, 1, H, D, generator=g).repeat_interleave(64, dim=2).reshape(B, S, H, D)
    return x.to(dtype).to(DEV)


def _order(B, H, S, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(S, generator=g) for _ in range(B * H)]).to(DEV)


def _bytes(t):
    return t.view(torch.uint8)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("stack", ["q_full", "q_plain_had", "k_smooth_perm_had", "k_plain", "q_mx_had", "k_mx_smooth"])
def test_q_and_k_chains(stack, D, dtype):
    B, S, H = 2, 512, 3
    x = _x(B, S, H, D, dtype, seed=hash((stack, D)) % 1000)
    order = _order(B, H, S, 7) if stack in ("q_full", "k_smooth_perm_had") else None
    smooth = 256 if stack == "q_full" else 0
    had = stack in ("q_plain_had", "k_smooth_perm_had", "q_mx_had")
    mean = k_channel_mean(x) if stack in ("k_smooth_perm_had", "k_mx_smooth") else None
    mx = stack in ("q_mx_had", "k_mx_smooth")
    signs = hadamard_signs(H, D, 3, DEV) if had else None
    # ---- the separate kernels
    w = _gather(x, order) if order is not None else x
    if mean is not None:
        w2, m2 = fq.smooth_k(x)
        assert torch.equal(m2, mean)
        w = _gather(w2, order) if order is not None else w2
    want_mean = None
    if smooth:
        w, want_mean = fq.group_mean_q(w, block_q=smooth)
    before_rotation = w
    if had:
        w, _ = fq.apply_qk_hadamard(w, w, random_sign=True, seed=3)
    s_pad = 640
    if mx:
        sf = torch.empty((B * H * s_pad * 4,), dtype=torch.uint8, device=DEV)
        wc, ws = fq.mxfp8_qk_quant(w, block_d=32, _layout=L.LAYOUT_BHSD, _s_pad=s_pad, _scale_e8=sf)
    else:
        wc, ws = fq.fp8_block_quant(w, block_s=64, _layout=L.LAYOUT_BHSD, _s_pad=s_pad)
    # ---- one fused pass
    gc, gs, gm, gsf, gprep = prep_fused(x, kind="mxfp8_qk" if mx else "fp8_block", scale_block=32 if mx else 64, order=order,
                                        chan_mean=mean, smooth_block=smooth, hadamard=had, signs=signs, layout=L.LAYOUT_BHSD,
                                        s_pad=s_pad, want_scale_e8=mx, want_prepared=True)
    raise_if_device_error(torch.device(DEV))
    assert torch.equal(_bytes(gc), _bytes(wc)) and torch.equal(gs, ws)
    assert torch.equal(gprep, before_rotation)
    if smooth:
        assert torch.equal(gm, want_mean)
    if mx:
        assert torch.equal(gsf, sf)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("kind", ["fp8_channel", "fp8_block", "mxfp8_v"])
@pytest.mark.parametrize("perm,smooth", [(True, 64), (False, 0), (True, 128), (False, 64)])
def test_v_chains(kind, perm, smooth, D, dtype):
    B, S, H = 2, 640, 2
    x = _x(B, S, H, D, dtype, seed=11)
    order = _order(B, H, S, 5) if perm else None
    w = _gather(x, order) if perm else x
    want_alpha = None
    if smooth:
        w, want_alpha = fq.smooth_v_per_block(w, block_s=smooth)
    s_pad = 640
    if kind == "fp8_channel":
        wc, ws = fq.fp8_per_channel_quant(w, _layout=L.LAYOUT_BHDS, _s_pad=s_pad)
    elif kind == "fp8_block":
        wc, ws = fq.fp8_block_quant(w, block_s=64, _layout=L.LAYOUT_BHDS, _s_pad=s_pad)
    else:
        wc, ws = fq.mxfp8_v_quant(w, block_s=64, _layout=L.LAYOUT_BHDS, _s_pad=s_pad)
    gc, gs, ga, _, _ = prep_fused(x, kind=kind, scale_block=0 if kind == "fp8_channel" else 64, order=order, smooth_block=smooth,
                                  layout=L.LAYOUT_BHDS, s_pad=s_pad)
    raise_if_device_error(torch.device(DEV))
    assert torch.equal(_bytes(gc), _bytes(wc)) and torch.equal(gs, ws)
    if smooth:
        assert torch.equal(ga, want_alpha)


def test_layouts_padding_and_refusals():
    x = _x(1, 192, 2, 128, torch.bfloat16, seed=2)
    wc, ws = fq.fp8_block_quant(x, block_s=64)
    gc, gs, _, _, _ = prep_fused(x, kind="fp8_block", scale_block=64)                                 # NHD
    assert torch.equal(_bytes(gc), _bytes(wc)) and torch.equal(gs, ws)
    gc, _, _, _, _ = prep_fused(x, kind="fp8_block", scale_block=64, layout=L.LAYOUT_BHSD, s_pad=256)
    assert int(_bytes(gc)[:, :, 192:].sum()) == 0 and torch.equal(_bytes(gc[:, :, :192].permute(0, 2, 1, 3).contiguous()), _bytes(wc))
    gc, _, _, _, _ = prep_fused(x, kind="fp8_block", scale_block=64, layout=L.LAYOUT_BHDS, s_pad=256)
    assert int(_bytes(gc)[..., 192:].sum()) == 0 and torch.equal(_bytes(gc[..., :192].permute(0, 3, 1, 2).contiguous()), _bytes(wc))
    assert group_rows("fp8_block", smooth_block=256, scale_block=64, seq=32768, dim=128, dtype=torch.bfloat16) == 256
    assert group_rows("fp8_channel", smooth_block=64, scale_block=0, seq=32768, dim=128, dtype=torch.bfloat16) == 128
    assert group_rows("fp8_block", smooth_block=4096, scale_block=64, seq=32768, dim=128, dtype=torch.float32) == 0   # no room
    with pytest.raises(ValueError, match="divisible"):
        prep_fused(x, kind="fp8_block", scale_block=80)
    with pytest.raises(NotImplementedError):
        prep_fused(_x(1, 4096, 1, 128, torch.float32, 1), kind="fp8_block", scale_block=64, smooth_block=4096)


CFGS = {
    "k_smooth_static": dict(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="elementwise"),
    "full_dynamic": dict(fp8_block_size=64, smoothing="full", q_kmeans_k=8, q_smooth_block_size=128, v_kmeans_k=8,
                         v_smooth_mode="per_block", v_smooth_block_size=64, p_quant="dynamic", rowmax_mode="qm_k"),
    "hadamard_full_vblock": dict(fp8_block_size=64, smoothing="full", q_kmeans_k=None, q_smooth_block_size=128, qk_hadamard=True,
                                 v_quant="fp8_block", v_smooth_mode="per_block"),
    "mx_general": dict(qk_quant="mxfp8", v_quant="fp8_block", qk_hadamard=True, smoothing="k_only", q_kmeans_k=4),
    "blasst": dict(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="dynamic", blasst_lambda=1e-2,
                   blasst_fill="mean_a1.5"),
}


@pytest.mark.parametrize("name", sorted(CFGS))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_entry_is_bit_identical_with_and_without_the_fused_path(name, dtype):
    cfg = QuantConfig(**CFGS[name])
    q, k, v = (_x(1, 512, 2, 128, dtype, seed=s) for s in (31, 32, 33))
    fused = fq.fake_quant_attention(q, k, v, cfg)
    with L.override(L.FLAG_UNFUSED_PREPROCESS):
        plain = fq.fake_quant_attention(q, k, v, cfg)
    raise_if_device_error(torch.device(DEV))
    assert torch.equal(fused, plain)
