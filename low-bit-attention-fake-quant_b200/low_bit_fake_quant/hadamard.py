"""Sign-randomised orthonormal Hadamard rotation of Q and K along D (CUDA).

API of src/low_bit_fake_quant/hadamard.py:15-124. The butterflies run in the
same order as the reference's torch FWHT (:25-47), in FP32, one warp per row;
the sign table comes from the same CPU generator (:58-62), so the rotation is
bit-identical to the reference's fallback path.
"""

from __future__ import annotations

import math
from functools import lru_cache
from typing import Callable

import torch

from . import _lib as L


def fast_hadamard_available() -> bool:
    """Whether the optional Dao-AILab CUDA op is in use: never -- the rotation
    is one of this library's own kernels."""
    return False


def _next_power_of_two(x: int) -> int:
    return 1 << (x - 1).bit_length()


def hadamard_transform_last_dim(x: torch.Tensor, *, scale: float, _signs: torch.Tensor | None = None,
                                _heads: int = 1) -> torch.Tensor:
    """Unstructured Hadamard transform over the final dimension (64 or 128)."""
    if not x.is_cuda:
        raise ValueError("hadamard_transform_last_dim expects a CUDA tensor")
    d = x.shape[-1]
    xc = x.contiguous()
    out = torch.empty_like(xc)
    rows = xc.numel() // d
    with torch.cuda.device(x.device):
        L.check(L.lib().lbfq_hadamard(xc.data_ptr(), L.dtype_code(xc.dtype), rows, _heads, d, L.ptr(_signs),
                                      float(scale), out.data_ptr(), L.stream_ptr(x.device)))
    return out


@lru_cache(maxsize=128)
def _cached_cpu_signs(h: int, d: int, seed: int) -> torch.Tensor:
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    signs = torch.randint(0, 2, (h, d), generator=gen, dtype=torch.int8)
    return signs.mul_(2).sub_(1)


def apply_qk_hadamard(
    q: torch.Tensor,
    k: torch.Tensor,
    *,
    random_sign: bool = True,
    seed: int = 0,
    transform: Callable[[torch.Tensor], torch.Tensor] | None = None,
    head_offset: int = 0,
    total_heads: int | None = None,
    _cross: bool = False,
) -> tuple[torch.Tensor, torch.Tensor]:
    """``x' = FWHT(x * sign[h]) / sqrt(D)`` for Q and K with the same signs.

    ``head_offset`` / ``total_heads`` (extensions) index the sign table by
    global head so that a heads shard reproduces the unsharded rotation.
    """
    same = q.shape == k.shape or (_cross and q.ndim == k.ndim == 4 and q.shape[0] == k.shape[0] and q.shape[2:] == k.shape[2:])
    if not same:                                         # `_cross` (extension): K may have its own length
        raise ValueError(f"q/k shapes must match; got {tuple(q.shape)} and {tuple(k.shape)}")
    if q.ndim != 4:
        raise ValueError(f"q/k must be NHD tensors; got {tuple(q.shape)}")
    if not (q.is_cuda and k.is_cuda):
        raise ValueError("q/k Hadamard rotation expects CUDA tensors")
    _, _, h, d = q.shape
    if d <= 0:
        raise ValueError("head dimension must be positive")
    scale = 1.0 / math.sqrt(float(_next_power_of_two(d)))
    signs = None
    if random_sign:
        table = _cached_cpu_signs(total_heads if total_heads is not None else h, d, seed)
        signs = table[head_offset:head_offset + h].contiguous().to(q.device)
    if transform is not None:
        qw, kw = q.contiguous(), k.contiguous()
        if signs is not None:
            qw = qw * signs.view(1, 1, h, d).to(q.dtype)
            kw = kw * signs.view(1, 1, h, d).to(k.dtype)
        return transform(qw), transform(kw)
    return (hadamard_transform_last_dim(q, scale=scale, _signs=signs, _heads=h),
            hadamard_transform_last_dim(k, scale=scale, _signs=signs, _heads=h))


__all__ = ["apply_qk_hadamard", "fast_hadamard_available", "hadamard_transform_last_dim"]
