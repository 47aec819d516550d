"""Parity at the benchmark's own shapes and on the benchmark's own inputs.

One head of each benchmark stack at the full sequence length (S = 32760 padded to 32768 by the hook's rule), built by
``bench.py``'s input generators (outlier channels x10, K channel offset ~ N(0, 3): logit standard deviation ~ 18, or
the spatially local video-like tokens), through the library and through the CPU oracle with the same k-means labels:

* the reference-operand mode against the oracle in the reference's convention (``faithful=True``), and the default
  FP8-code path against the oracle in the true-FP8 convention (``faithful=False``): cosine >= 0.99999 and the rows
  whose error exceeds 2e-3 x RMS must stay within the single-code-flip bound and within ``MAX_FLIP_ROWS`` = 1 % of
  the rows (measured on these inputs: 3e-5 ... 3.9e-3, the largest on the dynamic-P stack);
* both paths reproduce the oracle's MSE and cosine against BF16 SDPA to within 1 % (what the reference's result
  tables report).
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench                                                           # noqa: E402
import low_bit_fake_quant as fq                                        # noqa: E402
from low_bit_fake_quant.attention_triton import raise_if_device_error  # noqa: E402
from low_bit_fake_quant.config import QuantConfig                      # noqa: E402
from low_bit_fake_quant.kmeans import kmeans_labels                    # noqa: E402
from oracle import api as OA                                           # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLIP_ROWS = float(os.environ.get("LBFQ_TEST_MAX_FLIP_ROWS", "0.01"))

STACKS = ["wan14b_self_attn_k_smooth_static", "wan14b_self_attn_full_dynamic", "wan14b_self_attn_mxfp8_hadamard",
          "wan14b_video_blasst_mean_1e-2"]


def _flip_stats(got, want, q, k, v, sm_scale):
    """parity_report needs the S x S softmax of the head to bound single-code flips: done in row chunks."""
    got, want = got.float(), want.float()
    rms = want.pow(2).mean().sqrt().item()
    row_err = (got - want).abs().amax(dim=-1)                                       # (1, S, 1)
    qf, kf = q.float()[0, :, 0], k.float()[0, :, 0]
    w_max = torch.empty(qf.shape[0])
    for r0 in range(0, qf.shape[0], 4096):
        sc = (qf[r0:r0 + 4096] @ kf.t()) * sm_scale
        w_max[r0:r0 + 4096] = torch.softmax(sc, dim=-1).amax(dim=-1)
    tol = 2e-3 * rms
    bound = tol + 2.0 * 0.125 * (2.0 * w_max).clamp_max(1.0) * v.float().abs().max().item()
    flip = row_err[0, :, 0] > tol
    a, b = got.double().flatten(), want.double().flatten()
    cos = float(torch.dot(a, b) / (a.norm() * b.norm()))
    return {"cos": cos, "flip_rows": flip.float().mean().item(), "over_bound": int((row_err[0, :, 0] > bound).sum()),
            "max_abs_over_rms": float((a - b).abs().max()) / rms}


@pytest.mark.parametrize("name", STACKS)
def test_one_head_at_the_benchmark_shape(name):
    cfg = QuantConfig(**bench.WORKLOADS[name][0])
    maker = bench.make_video_inputs if name.startswith("wan14b_video") else bench.make_inputs
    q, k, v = maker(1, 1, bench.S_REAL, bench.D_HEAD, 1234, DEV)
    q, k, v, pad = bench.pad_like_hook(q, k, v, cfg)
    assert q.shape[1] == 32768
    kw, okw = {}, {}
    if cfg.q_kmeans_k is not None:
        kw["_q_labels"] = kmeans_labels(q, n_clusters=cfg.q_kmeans_k)
        okw["q_labels"] = kw["_q_labels"].cpu().long()
    if cfg.v_kmeans_k is not None:
        kw["_v_labels"] = kmeans_labels(v, n_clusters=cfg.v_kmeans_k)
        okw["v_labels"] = kw["_v_labels"].cpu().long()
    sm = 1.0 / (bench.D_HEAD ** 0.5)
    sdpa = fq.reference_attention(q, k, v).float().cpu()
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    torch.set_num_threads(os.cpu_count() or 1)
    report = {}
    for mode, extra, faithful in (("fp8_codes", {}, False), ("reference_operands", {"_reference_operands": True}, True)):
        got = fq.fake_quant_attention(q, k, v, cfg, _debug_fp32=True, **kw, **extra).float().cpu()
        raise_if_device_error(torch.device(DEV))
        # P convention of the kernel that ran: the TMEM-resident kernel rounds the re-scaled P to BF16 as the reference
        # does; the general kernel (here: BLASST on the reference's operands) applies the P scale in FP32
        want = OA.fake_quant_attention(qc, kc, vc, cfg, faithful=faithful, out_fp32=True, p_bf16=_p_bf16(cfg), **okw)
        st = _flip_stats(got, want, qc, kc, vc, sm)
        a, b = OA.compute_metrics(got, sdpa), OA.compute_metrics(want, sdpa)
        st.update(mse_vs_sdpa=a["mse"], mse_vs_sdpa_oracle=b["mse"], cos_vs_sdpa=a["cosine"], cos_vs_sdpa_oracle=b["cosine"])
        report[mode] = st
    print(f"\\n[baseline-shape parity] {name}: {report}")
    for mode, st in report.items():
        assert st["cos"] >= 0.99999, (name, mode, st)
        assert st["over_bound"] == 0 and st["flip_rows"] <= MAX_FLIP_ROWS, (name, mode, st)
        assert abs(st["mse_vs_sdpa"] / st["mse_vs_sdpa_oracle"] - 1.0) < 0.01, (name, mode, st)
        assert abs((1 - st["cos_vs_sdpa"]) / (1 - st["cos_vs_sdpa_oracle"]) - 1.0) < 0.01, (name, mode, st)


def _p_bf16(cfg):
    """Which P convention the default path's kernel uses: the TMEM-resident kernel hands scaled P to a BF16 P.V as the
    reference rounds it; the general kernel (BLASST with dynamic P on these stacks goes to the TMEM-resident one too)
    applies the scale in FP32."""
    from low_bit_fake_quant import _lib as L
    return L.lib().lbfq_attention_last_variant() == 1 and cfg.p_requant


def _e4m3_neighbours(c):
    """Next lower / higher e4m3 value of non-negative e4m3 values (FP32 tensors)."""
    bits = c.to(torch.float8_e4m3fn).view(torch.uint8).to(torch.int16)
    dn = (bits - 1).clamp(0, 0x7E).to(torch.uint8).view(torch.float8_e4m3fn).float()
    up = (bits + 1).clamp(0, 0x7E).to(torch.uint8).view(torch.float8_e4m3fn).float()
    return dn, up


def _bf16_neighbours(x):
    """Next lower / higher BF16 value of positive BF16 values (FP32 tensors)."""
    bits = x.to(torch.bfloat16).view(torch.int16)
    return (bits - 1).view(torch.bfloat16).float(), (bits + 1).view(torch.bfloat16).float()


@pytest.mark.parametrize("name", ["wan14b_self_attn_k_smooth_static", "wan14b_self_attn_full_dynamic"])
def test_rows_outside_the_tolerance_are_single_rounding_flips(name):
    """The rows of the previous test that exceed 2e-3 x RMS are claimed to differ from the oracle by ONE rounding
    decision of a P value that sits on a rounding boundary: an e4m3 code step, or -- in the scaled P modes, where the
    reference rounds ``p_fp8 x s_P`` to BF16 before P.V (attention_triton.py:353-360) -- one BF16 ulp of a heavy P
    value (the rows concerned are strongly peaked: one key carries most of the weight, and one BF16 ulp of its P is
    2^-8 of the row). Checked here on the worst rows: the oracle recomputes the row with one such value moved to its
    neighbour, and the kernel's row must then be within the tolerance (a second move is allowed for, a third is not).
    The oracle is run on the row alone, which is itself a slightly different summation order from the full run."""
    cfg = QuantConfig(**bench.WORKLOADS[name][0])
    q, k, v = bench.make_inputs(1, 1, bench.S_REAL, bench.D_HEAD, 1234, DEV)
    q, k, v, _ = bench.pad_like_hook(q, k, v, cfg)
    kw, okw = {}, {}
    inv = None
    if cfg.q_kmeans_k is not None:
        kw["_q_labels"] = kmeans_labels(q, n_clusters=cfg.q_kmeans_k)
        okw["q_labels"] = kw["_q_labels"].cpu().long()
        inv = OA.reorder_from_labels(q.cpu(), okw["q_labels"]).inverse_order[0]
    if cfg.v_kmeans_k is not None:
        kw["_v_labels"] = kmeans_labels(v, n_clusters=cfg.v_kmeans_k)
        okw["v_labels"] = kw["_v_labels"].cpu().long()
    got = fq.fake_quant_attention(q, k, v, cfg, _debug_fp32=True, **kw).float().cpu()
    raise_if_device_error(torch.device(DEV))
    p_bf16 = bool(_p_bf16(cfg)) and cfg.p_quant != "elementwise"
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    torch.set_num_threads(os.cpu_count() or 1)
    common = dict(faithful=False, out_fp32=True, p_bf16=p_bf16, **okw)
    want = OA.fake_quant_attention(qc, kc, vc, cfg, **common)
    tol = 2e-3 * want.pow(2).mean().sqrt().item()
    row_err = (got - want).abs().amax(dim=-1)[0, :, 0]
    flagged = torch.nonzero(row_err > tol).flatten()
    if flagged.numel() == 0:
        pytest.skip("no row outside the tolerance on these inputs")
    worst = flagged[torch.argsort(row_err[flagged], descending=True)][:3]
    explained = []
    for r in worst.tolist():
        pos = torch.tensor([int(inv[r]) if inv is not None else r])
        moves = []
        for _ in range(2):                                       # at most two moves per row
            probe = {}
            base = _with_moves(qc, kc, vc, cfg, common, pos, moves, probe)
            if (got[0, r, 0] - base).abs().max().item() <= tol:
                break
            x, c = probe["quotient"][0, 0, 0], probe["codes"][0, 0, 0]
            dn, up = _e4m3_neighbours(c)
            # distance of the quotient to the two rounding boundaries of its code, in code steps
            d_up = ((c + up) / 2 - x).abs() / (up - c).clamp_min(1e-30)
            d_dn = (x - (c + dn) / 2).abs() / (c - dn).clamp_min(1e-30)
            d = torch.minimum(torch.where(up > c, d_up, torch.full_like(x, 9.0)), torch.where(c > dn, d_dn, torch.full_like(x, 9.0)))
            # weight of each P value in the row's result (up to the common 1 / l): its value, brought to the row's last
            # reference max
            m_row = probe["row_max"][0, 0, 0]
            weight = probe["p_used"][0, 0, 0] * torch.exp2((m_row - m_row[-1]) * 1.4426950408889634)
            near = torch.nonzero(d < 5e-3).flatten()              # within 1/200 of a code step of a boundary
            near = near[torch.argsort(weight[near], descending=True)][:6]
            cands = [((n, 1 if d_up[n] <= d_dn[n] else -1), float(d[n]), "e4m3") for n in near.tolist()]
            if p_bf16:
                ps, pu = probe["p_scaled"][0, 0, 0], probe["p_used"][0, 0, 0]
                lo, hi = _bf16_neighbours(pu)
                for n in torch.argsort(weight, descending=True)[:3].tolist():     # the three heaviest values
                    for step, nb in ((1, hi[n]), (-1, lo[n])):
                        ulp = abs(float(nb - pu[n]))
                        dist = abs(float(ps[n]) - (float(pu[n]) + float(nb)) / 2) / max(ulp, 1e-30)
                        cands.append(((n, step, "bf16"), dist, "bf16"))
            best = None
            for move, dist, kind in cands:
                cand = _with_moves(qc, kc, vc, cfg, common, pos, moves + [move], None)
                err = (got[0, r, 0] - cand).abs().max().item()
                if best is None or err < best[0]:
                    best = (err, move, dist, kind)
            assert best is not None, (name, r, "no P value of this row lies near a rounding boundary")
            moves.append(best[1])
            explained.append({"row": r, "key": best[1][0], "step": best[1][1], "rounding": best[3],
                              "boundary_distance_in_steps": best[2], "heaviest_weight": float(weight.max() / weight.sum()),
                              "error_over_tol_before": row_err[r].item() / tol, "after": best[0] / tol})
        final = _with_moves(qc, kc, vc, cfg, common, pos, moves, None)
        assert (got[0, r, 0] - final).abs().max().item() <= tol, (name, explained)
        assert len(moves) <= 2
    print(f"\n[rows outside the tolerance] {name}: {int(flagged.numel())} of {row_err.numel()}; worst explained by: {explained}")
    # the values that were moved sat within 1/200 of a step of the rounding boundary in question
    assert all(e["boundary_distance_in_steps"] < 5e-3 for e in explained), explained


def _with_moves(qc, kc, vc, cfg, common, pos, moves, probe):
    """Row ``pos`` (kernel row order) of the oracle with the listed rounding moves applied."""
    flips = [(0,) + tuple(m) for m in moves] or None
    return OA.fake_quant_attention(qc, kc, vc, cfg, rows=pos, p_probe=probe, p_flip=flips, **common)[0, 0, 0]
