"""The CPU oracle against vectors produced by the reference itself.

``tests/golden/reference_cpu_vectors.pt`` was written by
``tests/golden/make_golden.py`` from the reference's CPU-runnable code: its
torch FWHT and sign generator, its row-max estimate, its fill-string parser,
the torch mirrors its own tests hold for the streaming kernel, and its
orchestration glue. These pin ``oracle/`` before the oracle is trusted as the
checker of the CUDA path.
"""
import math

import pytest
import torch

from low_bit_fake_quant.attention_triton import _parse_blasst_fill
from low_bit_fake_quant.config import QuantConfig
from oracle import api as OA
from oracle import quant_ops as OQ
from oracle.k12 import k12_attention, parse_blasst_fill


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten()[None], b.float().flatten()[None]).item()


def test_hadamard_matches_reference_fwht_bit_exact(golden):
    for key, d in (("hadamard_d128", 128), ("hadamard_d64", 64)):
        x, y = golden[key]["x"], golden[key]["y"]
        got = OQ.hadamard_transform_last_dim(x, scale=1.0 / math.sqrt(d))
        assert got.dtype == y.dtype and torch.equal(got, y), key


def test_sign_table_matches_reference_generator(golden):
    assert torch.equal(OQ.qk_signs(6, 128, 0), golden["signs"]["h6_d128_s0"])
    assert torch.equal(OQ.qk_signs(3, 64, 7), golden["signs"]["h3_d64_s7"])


def test_rowmax_estimate_matches_reference(golden):
    g = golden["rowmax_qm_k"]
    got = OA.estimate_rowmax_from_qm_k(g["qm"], g["k"], block_q=g["block_q"], sm_scale=g["sm_scale"])
    assert got.shape == g["y"].shape
    torch.testing.assert_close(got, g["y"], rtol=1e-5, atol=1e-5)


def test_fill_parser_matches_reference(golden):
    for mode, want in golden["parse_fill"]:
        assert parse_blasst_fill(mode, alpha=0.75, uta_bins=8) == tuple(want), mode
        assert _parse_blasst_fill(mode, alpha=0.75, uta_bins=8) == tuple(want), mode
    with pytest.raises(ValueError):
        parse_blasst_fill("bogus", alpha=1.0, uta_bins=8)
    with pytest.raises(ValueError):
        _parse_blasst_fill("bogus", alpha=1.0, uta_bins=8)


def test_k12_matches_reference_elementwise_mirror(golden):
    """Same bound as the reference's own kernel-vs-mirror test
    (tests/test_triton_attn.py:172-175): cos > 0.999, max-abs < 5e-2."""
    g = golden["mirror_elementwise"]
    D = g["q"].shape[-1]
    out = k12_attention(g["q"].float(), g["k"].float(), g["v"].float(), g["v_scale"], sm_scale=1.0 / math.sqrt(D),
                        p_max_offset=8, block_m=64, block_n=64, faithful=True).to(torch.bfloat16)
    assert _cos(out, g["y"]) > 0.999
    assert (out.float() - g["y"].float()).abs().max().item() < 5e-2


@pytest.mark.parametrize("mode", ["max_a0.25", "mean_a1.5", "logn", "sample8_a1.25", "thr_a0.25", "uta16_a1.5"])
def test_k12_matches_reference_blasst_mirror(golden, mode):
    """The BLASST mirror walks the same 32-key blocks, so agreement is far
    tighter than the reference's own bound (cos > 0.999, max-abs < 7e-2)."""
    g = golden["mirror_blasst"]
    B, H, S, D = g["q"].shape
    out, stats = k12_attention(g["q"].float(), g["k"].float(), g["v"].float(), torch.ones(B, H, D),
                               sm_scale=1.0 / math.sqrt(D), p_max_offset=8, block_m=32, block_n=32,
                               blasst_lambda=g["lam"], blasst_fill_mode=mode, faithful=True, return_stats=True)
    want = g["fills"][mode]
    assert stats[..., 0].sum().item() > 0
    assert stats.shape == (S // 32, B * H, 2)
    assert _cos(out, want) > 0.99999
    assert (out.to(torch.bfloat16).float() - want.float()).abs().max().item() < 2e-2


def test_orchestration_matches_reference_glue(golden):
    """oracle.api against the reference's _preprocess / _fake_quant_attention_*
    glue run on CPU (kernels swapped for the restatements on both sides)."""
    g = golden["glue"]
    for case in g["cases"]:
        cfg = QuantConfig(**case["cfg"])
        got = OA.fake_quant_attention(g["q"], g["k"], g["v"], cfg, faithful=True)
        want = case["out"]
        assert got.shape == want.shape and got.dtype == want.dtype
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 1e-6, (case["cfg"], diff)
