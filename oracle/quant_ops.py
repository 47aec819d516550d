"""CPU restatement of the reference quantizers and preprocess kernels.

TEST INFRASTRUCTURE ONLY. Nothing under ``oracle/`` is part of the shipped
path: only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU
baseline legs import it, and only as the checker / CPU baseline.

Every function restates, in plain torch on CPU tensors, one Triton kernel of
the reference (paths relative to the reference project root):

* ``fp8_block_quant`` / ``_dequant``        src/low_bit_fake_quant/quant_triton.py:26-131
* ``fp8_per_channel_quant`` / ``_dequant``  quant_triton.py:134-218
* ``mxfp8_qk_quant`` / ``_dequant``         quant_triton.py:221-319
* ``mxfp8_v_quant`` / ``_dequant``          quant_triton.py:322-416
* ``smooth_k``                              src/low_bit_fake_quant/preprocess.py:10-57
* ``group_mean_q``                          preprocess.py:60-91,169-193
* ``smooth_v_per_block``                    preprocess.py:94-166
* ``hadamard_transform_last_dim`` / ``apply_qk_hadamard``
                                            src/low_bit_fake_quant/hadamard.py:25-117

Pinning. The reference holds no golden vectors for codes or scales, so they
were recorded from its own Triton kernels run on a B200
(``tests/golden/make_golden_gpu.py`` -> ``tests/golden/reference_gpu_vectors.pt``)
and this module is held to them by ``tests/test_oracle_vs_reference_gpu.py``.
What the recording showed, and the arithmetic contract that follows from it:

* Triton's ``/`` is not an IEEE division: on the GPU ``a / b`` is exactly
  ``a * rcp.approx(b)`` (``div.full.f32``). With the constant divisor 448 that is
  ``amax * fl32(1/448)``, which a CPU reproduces bit for bit: every scale below is
  formed that way (an IEEE ``amax / 448`` differs by one ulp in half of the scales).
* ``x / scale`` uses the GPU's approximate reciprocal of ``scale``, a table a CPU
  cannot restate; the IEEE quotient used here rounds to the same e4m3 code except
  where the two land on opposite sides of a rounding boundary -- measured: 3 codes
  in 4.2 M. The CUDA library follows the GPU arithmetic and is bit-identical to
  the recorded codes; tests against this module allow that rate.
* fp32 -> e4m3 is round-to-nearest-even with saturation to +-448 (the GPU's
  ``cvt.rn.satfinite``; torch's CPU cast returns NaN above 448, hence the clamp in
  :func:`to_e4m3`); the power-of-two scale ``2**ceil(log2(amax/448))`` is taken by
  exact exponent arithmetic on ``amax * fl32(1/448)`` (identical to the recorded
  scales; ``fl32(1/448) * 1.75 * 2**j`` rounds to ``2**(j-8)`` exactly).
* the means of the smoothing kernels are fp32 sums in an unspecified tree order
  on the GPU; the recorded means differ from the sequential sums here by one ulp
  in under 1 % of the entries, the smoothed tensors not at all.

The pieces of the reference that run on CPU (its torch FWHT, the sign generator,
the row-max estimate, the SDPA glue and the torch mirrors in its own tests) pin
this module through ``tests/golden/reference_cpu_vectors.pt`` as well.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

FP8_MAX = 448.0
# fl32(1/448): what the GPU's ``amax / 448`` multiplies by (see the module docstring)
INV_FP8_MAX = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(448.0, dtype=torch.float32)
AMAX_FLOOR = 1e-4
UE8M0_MIN = -127
UE8M0_MAX = 127


# --------------------------------------------------------------------------
# element helpers
# --------------------------------------------------------------------------

# The reference's ``a / b`` is ``a * rcp.approx(b)`` on the GPU (module docstring). A test that has a GPU at hand can
# install that reciprocal (``low_bit_fake_quant._lib.rcp_approx``) and the restatement then follows the GPU arithmetic
# bit for bit; without it the IEEE quotient is used.
_RECIPROCAL = None


def set_reciprocal(fn) -> None:
    """``fn``: fp32 CPU tensor -> its element-wise reciprocal as the GPU's ``rcp.approx.f32`` returns it, or None."""
    global _RECIPROCAL
    _RECIPROCAL = fn


def divide(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """The reference kernels' ``a / b`` (``b`` broadcasts against ``a``)."""
    if _RECIPROCAL is None:
        return a / b
    return a * _RECIPROCAL(b.float().contiguous()).reshape(b.shape)


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 codes, round-to-nearest-even, saturating at +-448."""
    return x.float().clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def _fp32(x: float) -> float:
    return float(torch.tensor(x, dtype=torch.float32))


def pow2_scale(amax: torch.Tensor) -> torch.Tensor:
    """``2**clamp(ceil(log2(amax/448)), -127, 127)`` as fp32, exactly.

    quant_triton.py:240-243. ``amax`` is already floored at 1e-4. The
    quotient is ``amax * fl32(1/448)`` as on the GPU; ``ceil(log2(r))`` of an
    fp32 ``r`` is its exponent, minus one when ``r`` is itself a power of two.
    """
    r = amax.float() * INV_FP8_MAX
    mant, expo = torch.frexp(r)            # r = mant * 2**expo, mant in [0.5, 1)
    e = torch.where(mant == 0.5, expo - 1, expo)
    e = e.clamp(UE8M0_MIN, UE8M0_MAX).to(torch.float32)
    return torch.exp2(e)


def _check_nhd(t: torch.Tensor) -> Tuple[int, int, int, int]:
    if t.ndim != 4:
        raise ValueError(f"tensor must be 4-D NHD (B, S, H, D); got {tuple(t.shape)}")
    b, s, h, d = t.shape
    if d not in (64, 128):
        raise ValueError(f"tensor.shape[-1] must be 64 or 128; got {d}")
    return b, s, h, d


# --------------------------------------------------------------------------
# quantizers
# --------------------------------------------------------------------------

def fp8_block_quant(t: torch.Tensor, block_s: int = 128):
    """One FP32 scale per (B, S/block_s, H). quant_triton.py:26-77."""
    b, s, h, d = _check_nhd(t)
    if s % block_s != 0:
        raise ValueError(f"S={s} must be divisible by block_s={block_s}")
    n = s // block_s
    x = t.float().reshape(b, n, block_s, h, d)
    amax = x.abs().amax(dim=(2, 4)).clamp_min(AMAX_FLOOR)          # (b, n, h)
    sc = amax * INV_FP8_MAX
    codes = to_e4m3(divide(x, sc[:, :, None, :, None])).reshape(b, s, h, d)
    return codes, sc


def fp8_block_dequant(fp8, scale, block_s: int = 128, *, dtype=torch.float32):
    """quant_triton.py:80-131: ``code.fp32 * sc`` stored in ``dtype``."""
    b, s, h, d = _check_nhd(fp8)
    x = fp8.float().reshape(b, s // block_s, block_s, h, d) * scale.float()[:, :, None, :, None]
    return x.reshape(b, s, h, d).to(dtype)


def fp8_per_channel_quant(t: torch.Tensor, block_s: int = 128):
    """One FP32 scale per (B, H, D) over all of S. quant_triton.py:134-176."""
    b, s, h, d = _check_nhd(t)
    x = t.float()
    amax = x.abs().amax(dim=1).clamp_min(AMAX_FLOOR)               # (b, h, d)
    sc = amax * INV_FP8_MAX
    codes = to_e4m3(divide(x, sc[:, None]))
    return codes, sc


def fp8_per_channel_dequant(fp8, scale, block_s: int = 128, *, dtype=torch.float32):
    """quant_triton.py:179-218."""
    return (fp8.float() * scale.float()[:, None]).to(dtype)


def mxfp8_qk_quant(t: torch.Tensor, block_d: int = 32):
    """Power-of-two scale per (B, S, H, D/block_d). quant_triton.py:221-271."""
    b, s, h, d = _check_nhd(t)
    if d % block_d != 0:
        raise ValueError(f"D={d} must be divisible by block_d={block_d}")
    nb = d // block_d
    x = t.float().reshape(b, s, h, nb, block_d)
    amax = x.abs().amax(dim=-1).clamp_min(AMAX_FLOOR)              # (b, s, h, nb)
    sc = pow2_scale(amax)
    codes = to_e4m3(x / sc[..., None]).reshape(b, s, h, d)
    return codes, sc


def mxfp8_qk_dequant(fp8, scale, block_d: int = 32, *, dtype=torch.float32):
    """quant_triton.py:274-319."""
    b, s, h, d = _check_nhd(fp8)
    x = fp8.float().reshape(b, s, h, d // block_d, block_d) * scale.float()[..., None]
    return x.reshape(b, s, h, d).to(dtype)


def mxfp8_v_quant(t: torch.Tensor, block_s: int = 32):
    """Power-of-two scale per (B, S/block_s, H, D): blocks run along S.

    quant_triton.py:322-369.
    """
    b, s, h, d = _check_nhd(t)
    if s % block_s != 0:
        raise ValueError(f"S={s} must be divisible by block_s={block_s}")
    n = s // block_s
    x = t.float().reshape(b, n, block_s, h, d)
    amax = x.abs().amax(dim=2).clamp_min(AMAX_FLOOR)               # (b, n, h, d)
    sc = pow2_scale(amax)
    codes = to_e4m3(x / sc[:, :, None]).reshape(b, s, h, d)
    return codes, sc


def mxfp8_v_dequant(fp8, scale, block_s: int = 32, *, dtype=torch.float32):
    """quant_triton.py:372-416."""
    b, s, h, d = _check_nhd(fp8)
    x = fp8.float().reshape(b, s // block_s, block_s, h, d) * scale.float()[:, :, None]
    return x.reshape(b, s, h, d).to(dtype)


# --------------------------------------------------------------------------
# smoothing (preprocess.py)
# --------------------------------------------------------------------------

def smooth_k(k: torch.Tensor, block_s: int = 256):
    """K - mean_S(K). preprocess.py:10-57.

    The reference accumulates fp32 partial sums over chunks of ``block_s``
    rows and divides by S; the result is stored in K's dtype (one rounding),
    the mean as fp32 (B, H, D).
    """
    b, s, h, d = k.shape
    x = k.float()
    acc = torch.zeros((b, h, d), dtype=torch.float32)
    for s0 in range(0, s, block_s):
        acc = acc + x[:, s0:s0 + block_s].sum(dim=1)
    mean = divide(acc, torch.tensor(float(s), dtype=torch.float32))
    return (x - mean[:, None]).to(k.dtype), mean


def _block_mean_sub(t: torch.Tensor, block: int):
    b, s, h, d = t.shape
    if s % block != 0:
        raise ValueError(f"S={s} must be divisible by block_s={block}")
    if d not in (64, 128):
        raise ValueError(f"D must be 64 or 128; got {d}")
    n = s // block
    x = t.float().reshape(b, n, block, h, d)
    mean = divide(x.sum(dim=2), torch.tensor(float(block), dtype=torch.float32))   # (b, n, h, d)
    out = (x - mean[:, :, None]).reshape(b, s, h, d).to(t.dtype)
    return out, mean


def group_mean_q(q: torch.Tensor, block_q: int = 256):
    """Q minus the column mean of its ``block_q``-row group. preprocess.py:60-91."""
    return _block_mean_sub(q, block_q)


def smooth_v_per_block(v: torch.Tensor, block_s: int = 64):
    """V minus the column mean of its ``block_s``-row block. preprocess.py:94-166."""
    return _block_mean_sub(v, block_s)


# --------------------------------------------------------------------------
# Hadamard rotation (hadamard.py)
# --------------------------------------------------------------------------

def _next_pow2(x: int) -> int:
    return 1 << (x - 1).bit_length()


def hadamard_transform_last_dim(x: torch.Tensor, *, scale: float) -> torch.Tensor:
    """Unnormalised Sylvester-ordered FWHT over the last dim, times ``scale``.

    hadamard.py:25-47: fp32 butterflies with strides 1, 2, 4, ...; the product
    with ``scale`` is rounded once into ``x.dtype``.
    """
    dim = x.shape[-1]
    n = _next_pow2(dim)
    y = x.float()
    if n != dim:
        y = torch.nn.functional.pad(y, (0, n - dim))
    shape = y.shape
    y = y.reshape(-1, n).clone()
    stride = 1
    while stride < n:
        y = y.reshape(-1, n // (2 * stride), 2, stride)
        left = y[:, :, 0, :].clone()
        right = y[:, :, 1, :].clone()
        y = torch.stack((left + right, left - right), dim=2).reshape(-1, n)
        stride *= 2
    y = (y.reshape(shape)[..., :dim] * float(scale)).to(x.dtype)
    return y.reshape(x.shape)


def qk_signs(h: int, d: int, seed: int) -> torch.Tensor:
    """+-1 table (H, D) from a CPU generator. hadamard.py:58-62."""
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    signs = torch.randint(0, 2, (h, d), generator=gen, dtype=torch.int8)
    return signs.mul_(2).sub_(1)


def apply_qk_hadamard(q, k, *, random_sign: bool = True, seed: int = 0,
                      head_offset: int = 0, total_heads: Optional[int] = None):
    """``x' = FWHT(x * sign[h]) / sqrt(D)`` for Q and K. hadamard.py:77-117.

    ``head_offset`` / ``total_heads`` select rows of the sign table by global
    head index so that a batch x heads shard reproduces the unsharded result.
    """
    _, _, h, d = q.shape
    qw, kw = q, k
    if random_sign:
        table = qk_signs(total_heads if total_heads is not None else h, d, seed)
        signs = table[head_offset:head_offset + h].view(1, 1, h, d)
        qw = q * signs.to(q.dtype)
        kw = k * signs.to(k.dtype)
    scale = 1.0 / math.sqrt(float(_next_pow2(d)))
    return (hadamard_transform_last_dim(qw, scale=scale).contiguous(),
            hadamard_transform_last_dim(kw, scale=scale).contiguous())
