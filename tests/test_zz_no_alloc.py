"""The allocation-free variant of smooth_k, called through the C ABI.

``lbfq_smooth_k_static`` serves callers that can hand the library inputs and
outputs but no scratch (a plugin living inside another framework's memory
pool, a caller in a region where device allocation is not allowed). Its
partial sums live in an array built into the library, so the test checks what
such a caller relies on: the same bytes as ``lbfq_smooth_k`` with caller
scratch, on two calls in a row (the second call reuses the array the first one
dirtied, with a different shape), and a clear refusal above the array's size.
The file name sorts last on purpose: a run that stops at the first failure
has then already run every other test.
"""
import pytest
import torch

from low_bit_fake_quant import _lib as L

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _both(k):
    b, s, h, d = k.shape
    lib = L.lib()
    stream = L.stream_ptr(k.device)
    out_a, out_b = torch.empty_like(k), torch.empty_like(k)
    mean_a = torch.empty((b, h, d), dtype=torch.float32, device=k.device)
    mean_b = torch.empty_like(mean_a)
    n = lib.lbfq_smooth_k_scratch_floats(b, s, h, d)
    scratch = torch.empty((n,), dtype=torch.float32, device=k.device)
    L.check(lib.lbfq_smooth_k(k.data_ptr(), L.dtype_code(k.dtype), b, s, h, d, out_a.data_ptr(), mean_a.data_ptr(),
                              scratch.data_ptr(), stream))
    L.check(lib.lbfq_smooth_k_static(k.data_ptr(), L.dtype_code(k.dtype), b, s, h, d, out_b.data_ptr(),
                                     mean_b.data_ptr(), stream))
    torch.cuda.synchronize()
    return out_a, mean_a, out_b, mean_b


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    torch.manual_seed(0)
    with torch.cuda.device(DEV):
        for shape, dtype in (((2, 1000, 3, 128), torch.bfloat16), ((1, 300, 2, 64), torch.float16)):
            k = (torch.randn(*shape) + 2.0).to(dtype).to(DEV)
            out_a, mean_a, out_b, mean_b = _both(k)
            assert torch.equal(mean_a, mean_b)
            assert torch.equal(out_a, out_b)
            assert mean_b.abs().max() > 1.0          # it did compute something


def test_static_scratch_refuses_oversized_shapes():
    lib = L.lib()
    cap = lib.lbfq_smooth_k_static_max_floats()
    assert cap == 1 << 20
    b, s, h, d = 4, 32768, 40, 128                    # needs 4*40*128*128 floats > cap
    assert lib.lbfq_smooth_k_scratch_floats(b, s, h, d) > cap
    rc = lib.lbfq_smooth_k_static(None, L.BF16, b, s, h, d, None, None, None)
    assert rc == L.ERR_ARG
    assert b"built-in array" in lib.lbfq_last_error()
    with pytest.raises(ValueError):
        L.check(rc)


def test_static_scratch_mean_only_form():
    """``out = NULL`` asks for the channel mean alone (the form the K quantizer with fused smoothing uses): the same
    mean as the full call, and nothing else is written."""
    torch.manual_seed(1)
    with torch.cuda.device(DEV):
        k = (torch.randn(2, 777, 3, 128) + 1.5).bfloat16().to(DEV)
        b, s, h, d = k.shape
        _, mean_full, _, _ = _both(k)
        mean_only = torch.full((b, h, d), float("nan"), dtype=torch.float32, device=DEV)
        lib = L.lib()
        L.check(lib.lbfq_smooth_k_static(k.data_ptr(), L.dtype_code(k.dtype), b, s, h, d, None, mean_only.data_ptr(),
                                         L.stream_ptr(k.device)))
        torch.cuda.synchronize()
        assert torch.equal(mean_only, mean_full)
