"""Case list shared by ``make_golden_gpu.py`` (which runs the reference project's own Triton kernels on a GPU and
records what they return) and by the tests that hold the oracle and the CUDA library to those records.

Everything here is plain data + seeded input construction; nothing imports the reference.
"""
import math

import torch

# (S, H, D) of the operator-level cases and of the whole-entry cases
OP_SHAPES = ((256, 1, 128), (256, 2, 64))
ENTRY_SHAPE = (256, 2, 128)

# direct launches of the streaming kernel: name -> keyword description (see build_k12_operands / k12_kwargs)
K12_CASES = {
    "el_online": dict(p="elementwise"),
    "el_block32": dict(p="elementwise", block=32),
    "mx_vmx": dict(p="mx", v="mxfp8"),
    "dyn": dict(p="dynamic"),
    "dyn_valpha": dict(p="dynamic", v_smooth=64),
    "el_valpha": dict(p="elementwise", v_smooth=64),
    "el_vblock": dict(p="elementwise", v="fp8_block"),
    "dyn_vblock": dict(p="dynamic", v="fp8_block"),
    "dyn_qm": dict(p="dynamic", q_smooth=128),
    "dyn_qm_est": dict(p="dynamic", q_smooth=128, est=True),
    "el_qm_est": dict(p="elementwise", q_smooth=128, est=True),
    "mx_qm_est_valpha": dict(p="mx", v="mxfp8", q_smooth=128, est=True, v_smooth=64),
    "el_init": dict(p="elementwise", init=True),
    "bl_zero_el": dict(p="elementwise", lam=0.05, fill="zero"),
    "bl_max_dyn": dict(p="dynamic", lam=0.05, fill="max_a0.25"),
    "bl_mean_dyn": dict(p="dynamic", lam=0.05, fill="mean_a1.5"),
    "bl_logn_el": dict(p="elementwise", lam=0.05, fill="logn"),
    "bl_sample8_el": dict(p="elementwise", lam=0.05, fill="sample8_a1.25"),
    "bl_thr_mx": dict(p="mx", v="mxfp8", lam=0.05, fill="thr_a0.25"),
    "bl_uta16_dyn": dict(p="dynamic", lam=0.05, fill="uta16_a1.5"),
    "bl_uta4_el_vblock": dict(p="elementwise", v="fp8_block", lam=0.05, fill="uta4_a2"),
}
K12_CASES_D64 = ("el_online", "dyn_valpha", "dyn_qm_est")

# whole-entry configurations (QuantConfig keyword arguments); "labels" = which k-means label sets the case consumes
ENTRY_CASES = {
    "k_smooth_static": dict(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="elementwise"),
    "full_dynamic": dict(fp8_block_size=64, smoothing="full", q_kmeans_k=8, q_smooth_block_size=128, v_kmeans_k=8,
                         v_smooth_mode="per_block", v_smooth_block_size=64, p_quant="dynamic", rowmax_mode="qm_k"),
    "mxfp8_hadamard": dict(qk_quant="mxfp8", v_quant="mxfp8", mxfp8_block_size=32, v_mxfp8_block_size=64, qk_hadamard=True,
                           smoothing="off", q_kmeans_k=None, p_quant="auto"),
    "blasst_mean_dynamic": dict(fp8_block_size=64, smoothing="k_only", q_kmeans_k=None, p_quant="dynamic",
                                blasst_lambda=1e-2, blasst_fill="mean_a1.5"),
    "path_a_config1": dict(fp8_block_size=64, smoothing="off", q_kmeans_k=None, p_requant=False),
    "full_vblock_static": dict(fp8_block_size=64, v_quant="fp8_block", v_fp8_block_size=64, smoothing="full", q_kmeans_k=8,
                               q_smooth_block_size=128, p_quant="elementwise"),
    "path_a_full": dict(fp8_block_size=64, smoothing="full", q_kmeans_k=8, q_smooth_block_size=128, v_smooth_mode="per_block",
                        p_requant=False),
}


def base_inputs(seed: int, s: int, h: int, d: int, dtype=torch.bfloat16):
    """Seeded CPU tensors (1, S, H, D): N(0,1) with two channels scaled x4; K carries a per-channel offset."""
    g = torch.Generator().manual_seed(seed)
    scale = torch.ones(d)
    scale[3] = 4.0
    scale[d // 2 + 5] = 4.0
    q = torch.randn(1, s, h, d, generator=g) * scale
    k = torch.randn(1, s, h, d, generator=g) * scale + 1.5 * torch.randn(1, 1, h, d, generator=g)
    v = torch.randn(1, s, h, d, generator=g) + 0.5 * torch.randn(1, s // 64, 1, d, generator=g).repeat_interleave(64, dim=1)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def build_k12_operands(fq, q, k, v, spec, *, sm_scale):
    """The operands the reference's glue hands to its kernel (attention.py:531-608 of the reference), built with the
    quantizers / smoothing functions of ``fq`` -- the reference package when recording, this repository's package
    when replaying (both expose the same names). Returns (positional operands, keyword arguments)."""
    blk = spec.get("block", 64)
    to_bh = lambda t: t.permute(0, 2, 1, 3).contiguous()
    b, s, h, d = q.shape
    k_s, _ = fq.smooth_k(k)
    qm = None
    q_w = q
    if spec.get("q_smooth"):
        q_w, qm = fq.group_mean_q(q, block_q=spec["q_smooth"])
    v_w, v_alpha = v, None
    if spec.get("v_smooth"):
        v_w, v_alpha = fq.smooth_v_per_block(v, block_s=spec["v_smooth"])
    qc, qs = fq.fp8_block_quant(q_w, block_s=64)
    kc, ks = fq.fp8_block_quant(k_s, block_s=64)
    q_deq = fq.fp8_block_dequant(qc, qs, block_s=64, dtype=torch.bfloat16)
    k_deq = fq.fp8_block_dequant(kc, ks, block_s=64, dtype=torch.bfloat16)
    kw = dict(sm_scale=float(sm_scale), p_max_offset=8, block_m=blk, block_n=blk, p_quant_mode=spec["p"])
    vk = spec.get("v", "fp8_channel")
    if vk == "fp8_channel":
        vc, vs = fq.fp8_per_channel_quant(v_w)
        v_bf, v_scale = vc.to(torch.bfloat16), vs.float().contiguous()
    elif vk == "fp8_block":
        vc, vs = fq.fp8_block_quant(v_w, block_s=64)
        v_bf, v_scale = vc.to(torch.bfloat16), torch.ones((b, h, d), dtype=torch.float32, device=q.device)
        kw.update(v_block_scale_bsh=vs.float().contiguous(), v_block_size=64)
    else:
        vc, vs = fq.mxfp8_v_quant(v_w, block_s=64)
        v_bf = fq.mxfp8_v_dequant(vc, vs, block_s=64, dtype=torch.bfloat16)
        v_scale = torch.ones((b, h, d), dtype=torch.float32, device=q.device)
    if spec["p"] == "mx":
        kw.update(p_mx_block_n=blk)
    if v_alpha is not None:
        kw.update(v_alpha=v_alpha.float().contiguous(), v_smooth_block=spec["v_smooth"])
    if qm is not None:
        kw.update(k_smooth_bhsd=to_bh(k_s.to(torch.bfloat16)), qm_bhgd=qm.float().contiguous(), q_smooth_block=spec["q_smooth"])
    ops = (to_bh(q_deq), to_bh(k_deq), to_bh(v_bf), v_scale)
    if spec.get("est"):
        # attention.py:366-395 of the reference: max over keys of qm . K_smooth, one value per Q group, repeated per row
        qmb = qm.permute(0, 2, 1, 3).float()
        ksb = k_s.permute(0, 2, 1, 3).float()
        est = torch.matmul(qmb, ksb.transpose(-2, -1)).amax(dim=-1) * float(sm_scale)
        kw.update(rowmax_est_bhs=est.repeat_interleave(spec["q_smooth"], dim=2).contiguous())
    if spec.get("init"):
        # the diagonal initialisation of the reference's BLASST evaluation (bench/eval_blasst_quant.py:147-148)
        kw.update(rowmax_init_bhs=((ops[0].float() * ops[1].float()).sum(dim=-1) * float(sm_scale)).contiguous())
    if spec.get("lam") is not None:
        kw.update(blasst_lambda=spec["lam"], blasst_fill_mode=spec["fill"], return_blasst_stats=True)
    return ops, kw


def sm_scale_for(d: int) -> float:
    return 1.0 / math.sqrt(d)
