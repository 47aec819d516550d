"""pytest configuration: the ``gpu`` marker and import paths.

``-m "not gpu"`` runs the CPU suite (oracle vs golden vectors, host logic,
C-ABI symbol check, gloo sharding test); ``-m gpu`` runs the parity tests of
the CUDA library against the oracle on a B200.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "low-bit-attention-fake-quant_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_cpu_vectors.pt"), weights_only=False)


@pytest.fixture(autouse=True)
def _reset_debug_overrides():
    """Tests switch the library's debug overrides (general attention kernel, FFMA cross-check kernels) on and off;
    every test starts and ends with none of them set."""
    yield
    import torch

    if torch.cuda.is_available():
        from low_bit_fake_quant import _lib as L
        L.lib().lbfq_set_flags(0)


@pytest.fixture(autouse=True, scope="session")
def _oracle_follows_the_gpu_reciprocal():
    """With a GPU at hand the oracle divides as the GPU does (``a * rcp.approx(b)``, fetched through the library's
    test utility), so that quantizer codes can be compared bit for bit; without one it uses IEEE division."""
    import torch

    if torch.cuda.is_available():
        from low_bit_fake_quant import _lib as L
        from oracle import quant_ops as OQ
        OQ.set_reciprocal(lambda t: L.rcp_approx(t, device="cuda:0"))
    yield
