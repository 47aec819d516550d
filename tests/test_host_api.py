"""Host-side mirror of the reference API and the C-ABI boundary (no GPU needed)."""
import ctypes
import dataclasses
import os
import re

import pytest
import torch

import low_bit_fake_quant as fq
from low_bit_fake_quant import _lib as L
from low_bit_fake_quant.sharding import all_ranges, slab_range

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = L.lib()
    assert lib.lbfq_abi_version() >= 1
    header = open(os.path.join(ROOT, "include", "lbfq.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = sorted(set(re.findall(r"\b(lbfq_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/lbfq.h but not exported"
    assert sorted(L.exported_symbols()) == declared          # the ctypes table covers the whole header


def test_attn_args_struct_matches_header_field_order():
    header = open(os.path.join(ROOT, "include", "lbfq.h")).read()
    body = re.search(r"typedef struct lbfq_attn_args \{(.*?)\} lbfq_attn_args;", header, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for stmt in body.split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        for part in stmt.split(","):
            names.append(re.findall(r"([A-Za-z_][A-Za-z0-9_]*)\s*$", part.strip())[0])
    assert names == [f[0] for f in L.AttnArgs._fields_]


def test_public_names_match_reference_package():
    want = {"FakeQuantArtifacts", "KMeansReorderResult", "PreparedQKV", "PreprocessCache", "QuantConfig",
            "apply_qk_hadamard", "fake_quant_attention", "fast_hadamard_available", "prepare_for_attention",
            "fp8_block_dequant", "fp8_block_quant", "fp8_per_channel_dequant", "fp8_per_channel_quant",
            "group_mean_q", "hadamard_transform_last_dim", "smooth_v_per_block", "mxfp8_qk_dequant",
            "mxfp8_qk_quant", "mxfp8_v_dequant", "mxfp8_v_quant", "prepare_qkv", "apply_kv_permutation",
            "kmeans_reorder_tokens", "q_kmeans_reorder", "v_kmeans_reorder", "reference_attention", "smooth_k"}
    assert set(fq.__all__) == want
    for n in want:
        assert hasattr(fq, n)
    assert callable(fq.fake_quant_attention_host)             # extension, kept out of __all__


def test_quant_config_defaults_and_frozen():
    c = fq.QuantConfig()
    assert (c.qk_quant, c.v_quant, c.smoothing) == ("fp8_block", "fp8_channel", "full")
    assert (c.q_smooth_block_size, c.q_kmeans_k, c.q_kmeans_iters, c.q_kmeans_seed) == (256, 32, 10, 0)
    assert (c.fp8_block_size, c.mxfp8_block_size, c.v_fp8_block_size, c.v_mxfp8_block_size) == (128, 32, 64, 64)
    assert (c.p_quant, c.rowmax_mode, c.p_mx_block_n, c.p_max_offset, c.p_requant) == ("auto", "online", 0, 8, True)
    assert (c.p_requant_q_chunk, c.p_requant_block_m, c.p_requant_block_n) == (512, 64, 64)
    assert (c.blasst_lambda, c.blasst_fill, c.blasst_fill_alpha, c.blasst_uta_bins) == (None, "zero", 1.0, 16)
    assert (c.v_smooth_mode, c.v_smooth_block_size, c.v_kmeans_k, c.v_kmeans_iters, c.v_kmeans_seed) == ("off", 64, None, 10, 0)
    assert c.correction_dtype == torch.float16 and c.qk_hadamard is False and c.qk_hadamard_random_sign is True
    assert len(dataclasses.fields(c)) == 32
    with pytest.raises(dataclasses.FrozenInstanceError):
        c.qk_quant = "mxfp8"


def test_cpu_tensors_are_refused_like_the_reference():
    x = torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="must live on CUDA"):
        fq.fake_quant_attention(x, x, x)
    with pytest.raises(ValueError, match="must live on CUDA"):
        fq.fp8_block_quant(x)
    with pytest.raises(ValueError, match="on CUDA"):
        fq.smooth_k(x)
    with pytest.raises(ValueError, match="CUDA"):
        fq.apply_qk_hadamard(x, x)
    with pytest.raises(ValueError, match="on CUDA"):
        fq.kmeans_reorder_tokens(x, n_clusters=2)
    with pytest.raises(ValueError, match="4-D"):
        fq.fake_quant_attention(x[0], x[0], x[0])
    with pytest.raises(ValueError, match="shapes must match"):
        fq.fake_quant_attention(x, x[:, :32], x)


def test_c_abi_argument_errors_without_a_gpu():
    """Validation happens before any CUDA call, so it is observable on a CPU box."""
    lib = L.lib()
    rc = lib.lbfq_fp8_block_quant(None, L.BF16, 1, 100, 1, 128, 64, None, 0, 0, None, None)
    assert rc == L.ERR_ARG and b"divisible" in lib.lbfq_last_error()
    rc = lib.lbfq_fp8_block_quant(None, L.BF16, 1, 128, 1, 96, 64, None, 0, 0, None, None)
    assert rc == L.ERR_ARG and b"64 or 128" in lib.lbfq_last_error()
    with pytest.raises(ValueError):
        L.check(rc)
    a = L.AttnArgs()
    assert lib.lbfq_attention_fwd(ctypes.byref(a), None, None) == L.ERR_ARG
    # smooth_k's column-sum tiles are laid out for D = 64 / 128: any other head dimension is refused before a launch,
    # through both entries (the shape is checked before the size of the built-in scratch, and before any pointer)
    for d in (8, 32, 96, 256):
        rc = lib.lbfq_smooth_k(None, L.BF16, 1, 256, 1, d, None, None, None, None)
        assert rc == L.ERR_ARG and b"64 or 128" in lib.lbfq_last_error()
        rc = lib.lbfq_smooth_k_static(None, L.BF16, 1, 256, 1, d, None, None, None)
        assert rc == L.ERR_ARG and b"64 or 128" in lib.lbfq_last_error()
    # an unknown element type is a dtype error (TypeError in the host mirror) in every entry
    rc = lib.lbfq_fp8_block_quant(None, 7, 1, 128, 1, 128, 64, None, 0, 0, None, None)
    assert rc == L.ERR_DTYPE
    with pytest.raises(TypeError):
        L.check(rc)
    rc = lib.lbfq_gather_rows(None, 7, 1, 128, 1, 128, None, None, None)
    assert rc == L.ERR_DTYPE


def test_debug_flags_round_trip():
    lib = L.lib()
    before = L.flags()
    with L.override(L.FLAG_ATTN_GENERIC | L.FLAG_QM_CORR_FFMA):
        assert L.flags() & L.FLAG_ATTN_GENERIC and L.flags() & L.FLAG_QM_CORR_FFMA
        L.set_flag(L.FLAG_QM_CORR_FFMA, False)
        assert not (L.flags() & L.FLAG_QM_CORR_FFMA)
    assert L.flags() == before
    assert lib.lbfq_get_flags() == before


def test_flag_constants_match_the_header():
    header = open(os.path.join(ROOT, "include", "lbfq.h")).read()
    defined = {name: int(val) for name, val in re.findall(r"#define LBFQ_(FLAG_[A-Z_]+) (\d+)", header)}
    assert defined and all(getattr(L, name) == val for name, val in defined.items())
    assert len(set(defined.values())) == len(defined) and all(v & (v - 1) == 0 for v in defined.values())    # distinct bits


def test_host_entry_chunk_schedule():
    """The heads chunks of the host-buffer entry: default sizes, the tapered tail, an explicit schedule and its checks."""
    from low_bit_fake_quant.config import QuantConfig
    from low_bit_fake_quant.host import _chunk_bounds
    plain = QuantConfig(q_kmeans_k=None, v_kmeans_k=None)
    km = QuantConfig(q_kmeans_k=8, v_kmeans_k=None)
    for cfg, h in ((plain, 40), (km, 40), (plain, 5), (km, 3)):
        b = _chunk_bounds(h, cfg, None, None)
        assert b[0][0] == 0 and b[-1][1] == h and all(x[1] == y[0] for x, y in zip(b, b[1:])) and all(x[1] > x[0] for x in b)
    assert [hi - lo for lo, hi in _chunk_bounds(40, km, None, None)] == [2, 6, 8, 8, 8, 8]       # a short first chunk
    assert [hi - lo for lo, hi in _chunk_bounds(40, plain, None, None)][-3:] == [2, 1, 1]      # the tail tapers to one head
    assert _chunk_bounds(40, km, None, [2, 5, 10, 19, 4]) == [(0, 2), (2, 7), (7, 17), (17, 36), (36, 40)]
    for bad in ([], [40, 0], [20, 19], [41]):
        with pytest.raises(ValueError, match="chunk_heads"):
            _chunk_bounds(40, km, None, bad)
    with pytest.raises(ValueError, match="heads_per_chunk"):
        _chunk_bounds(40, km, 0, None)


def test_head_dimension_is_checked_before_any_launch():
    x = torch.zeros(1, 256, 1, 32, dtype=torch.bfloat16)

    class FakeCuda(torch.Tensor):
        """A CPU tensor that claims to live on CUDA: reaches the checks behind the device check without a GPU."""
        @property
        def is_cuda(self):
            return True

    y = x.as_subclass(FakeCuda)
    with pytest.raises(ValueError, match="64 or 128"):
        fq.fake_quant_attention(y, y, y, fq.QuantConfig(smoothing="k_only", q_kmeans_k=None))


def test_slab_ranges_partition_the_heads():
    for total in (40, 80, 7):
        for world in (1, 2, 4, 8):
            r = all_ranges(total, world)
            assert r[0][0] == 0 and r[-1][1] == total
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in r]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        slab_range(8, 2, 2)


def test_hook_padding_policy():
    """bench/wan_attention_hook.py:253-294 of the reference: pad to the lcm of the block sizes in play."""
    from low_bit_fake_quant.config import QuantConfig
    from low_bit_fake_quant.hook import pad_qkv, required_multiple
    cfg = QuantConfig(fp8_block_size=64, smoothing="full", q_smooth_block_size=256, v_smooth_mode="per_block",
                      v_smooth_block_size=96, q_kmeans_k=None)
    assert required_multiple(cfg) == 768                        # lcm(64, 64, 64, 64, 256, 96)
    assert required_multiple(QuantConfig(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None)) == 64
    q = torch.arange(2 * 100 * 1 * 4, dtype=torch.float32).view(2, 100, 1, 4)
    qp, kp, vp, pad = pad_qkv(q, q + 1, q + 2, QuantConfig(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None))
    assert pad == 28 and qp.shape == (2, 128, 1, 4)
    assert torch.equal(qp[:, :100], q) and qp[:, 100:].abs().sum() == 0
    assert torch.equal(kp[:, 100:], (q + 1)[:, -1:].expand(-1, 28, -1, -1))
    assert torch.equal(vp[:, 100:], (q + 2)[:, -1:].expand(-1, 28, -1, -1))
    same = pad_qkv(q[:, :64], q[:, :64], q[:, :64], QuantConfig(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None))
    assert same[3] == 0 and same[0] is not None and same[0].shape[1] == 64


def test_space_time_block_order():
    """bench/eval_blasst_quant.py:101-134 of the reference: bricks of (ts, hs, ws) tokens made contiguous."""
    from low_bit_fake_quant.hook import space_time_block_order
    t, h, w, ts, hs, ws = 4, 6, 8, 2, 3, 4
    order = space_time_block_order(t, h, w, ts=ts, hs=hs, ws=ws)
    ids = torch.arange(t * h * w).reshape(t // ts, ts, h // hs, hs, w // ws, ws)
    assert torch.equal(order, ids.permute(0, 2, 4, 1, 3, 5).reshape(-1))           # divisible grid: a reshape / permute
    # ragged grid + tail: still a permutation, the tail stays in place, every brick's tokens are contiguous
    t, h, w = 3, 5, 7
    order = space_time_block_order(t, h, w, ts=2, hs=2, ws=4, tail=5)
    n = t * h * w
    assert torch.equal(torch.sort(order).values, torch.arange(n + 5)) and torch.equal(order[n:], torch.arange(n, n + 5))
    tt, hh, ww = order[:n] // (h * w), (order[:n] // w) % h, order[:n] % w
    brick = ((tt // 2) * 3 + hh // 2) * 2 + ww // 4
    assert torch.equal(brick, torch.sort(brick, stable=True).values)               # bricks in order, never interleaved
    # the order the reference's block_shuffle_order returns for this ragged grid (generated from it)
    want = [0, 1, 3, 4, 2, 5, 6, 7, 8, 9, 10, 12, 13, 11, 14, 15, 16, 17, 18, 19]
    assert space_time_block_order(2, 3, 3, ts=1, hs=2, ws=2, tail=2).tolist() == want
    with pytest.raises(ValueError):
        space_time_block_order(0, 1, 1, ts=1, hs=1, ws=1)


def test_wan_hook_routing_log_dump_and_compare(tmp_path, monkeypatch):
    """bench/wan_attention_hook.py of the reference: routing by shape, call log, dump and compare switches. The
    fake-quant call itself needs a GPU; a CPU stand-in of the same signature takes its place here."""
    import types
    from low_bit_fake_quant import hook
    from low_bit_fake_quant.config import QuantConfig
    from oracle import api as OA

    calls = []

    def stand_in(q, k, v, cfg, *, sm_scale=None, preprocess_cache=None):
        calls.append((tuple(q.shape), cfg.rowmax_mode, preprocess_cache))
        return OA.reference_attention(q, k, v, sm_scale=sm_scale)

    monkeypatch.setattr(hook, "_attention_fn", stand_in)
    monkeypatch.setattr(hook, "_prepare_fn", lambda q, k, v, cfg: "cache")
    fake_wan = types.SimpleNamespace(attention=None, flash_attention=None)
    fake_model = types.SimpleNamespace(flash_attention=None)
    hook.install_hook(fake_wan, fake_model)
    assert fake_wan.attention is hook.wan_attention and fake_model.flash_attention is hook.wan_attention

    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1100, 2, 64, generator=g).bfloat16()
    text = torch.randn(1, 512, 2, 64, generator=g).bfloat16()
    cfg = QuantConfig(fp8_block_size=64, smoothing="full", q_smooth_block_size=256, q_kmeans_k=None, rowmax_mode="qm_k")
    # no configuration: everything is plain SDPA
    hook.set_quant_cfg(hook.NO_QUANT)
    ref = fake_wan.attention(q, q, q)
    fake_wan.attention(q, text, text)
    assert [r["kind"] for r in hook.get_call_log()] == ["self-sdpa", "cross-sdpa"] and not calls
    # with a configuration: self-attention is padded to the block sizes (lcm 256 -> 1280 rows), stripped and logged
    monkeypatch.setenv("WAN_ATTENTION_DUMP_DIR", str(tmp_path))
    monkeypatch.setenv("WAN_ATTENTION_COMPARE_SDPA", "1")
    monkeypatch.setenv("WAN_ATTENTION_COMPARE_ONLINE_ROWMAX", "1")
    hook.set_quant_cfg(cfg)
    assert hook.get_call_log() == []
    out = fake_wan.flash_attention(q.float(), q.float(), q.float(), softmax_scale=None, dtype=torch.bfloat16)
    fake_wan.attention(q, text, text)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    log = hook.get_call_log()
    assert [r["kind"] for r in log] == ["self-fq", "cross-sdpa"]
    assert log[0]["pad"] == 180 and log[0]["Lq"] == 1100 and log[0]["H"] == 2 and log[0]["D"] == 64
    assert calls[0] == ((1, 1280, 2, 64), "qm_k", "cache") and calls[1] == ((1, 1280, 2, 64), "online", "cache")
    assert set(log[0]["compare_sdpa"]) == {"mse", "cosine", "max_abs", "out_norm", "ref_norm", "out_has_nan", "out_has_inf"}
    assert log[0]["compare_online_rowmax"]["cosine"] > 0.999 and "ref_has_nan" in log[0]["compare_online_rowmax"]
    dumped = torch.load(log[0]["dumped_qkv"], weights_only=False)
    assert dumped["query"].shape == q.shape and dumped["record"]["kind"] == "self-fq"
    # the padded keys replicate the last token, so the stand-in's result is close to, not equal to, plain SDPA
    assert torch.nn.functional.cosine_similarity(out.float().flatten()[None], ref.float().flatten()[None]).item() > 0.99
    # the dump limit defaults to one call
    fake_wan.attention(q, q, q)
    assert "dumped_qkv" not in hook.get_call_log()[-1]
