"""Loader of the staged reference package (see ``oracle/make_ref.py``).

TEST INFRASTRUCTURE ONLY.

``load()`` returns the reference's package object, imported under the name
``ref_low_bit_fake_quant``, or ``None`` when it has not been staged or Triton
is missing. The reference imports the third-party ``flash_kmeans`` at module
level (kmeans.py:23), which is not installed here; a stand-in module is put in
``sys.modules`` whose ``batch_kmeans_Euclid`` hands back labels queued with
``inject_labels`` -- so a test can drive the reference's whole pipeline
(kmeans.py:77-95 sorts and gathers by whatever labels it is given) with the
same cluster assignment as the implementation under test.
"""
import importlib
import os
import sys
import types

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF_DIR = os.path.join(_HERE, "_ref")
_label_queue = []


def inject_labels(*labels):
    """Queue (B*H, S) label tensors for the reference's next k-means calls, in call order."""
    _label_queue.extend(labels)


def _batch_kmeans_stub(x, n_clusters, max_iters=10, tol=0.0, verbose=False):
    if not _label_queue:
        raise RuntimeError("reference k-means called with no labels injected (flash_kmeans is not installed)")
    lab = _label_queue.pop(0)
    assert tuple(lab.shape) == tuple(x.shape[:2]), (lab.shape, x.shape)
    return lab.to(device=x.device).to(dtype=__import__("torch").int32), None, max_iters


def load():
    if not os.path.isdir(os.path.join(_REF_DIR, "ref_low_bit_fake_quant")):
        return None
    try:
        import triton  # noqa: F401
    except Exception:
        return None
    if "flash_kmeans" not in sys.modules:
        stub = types.ModuleType("flash_kmeans")
        stub.batch_kmeans_Euclid = _batch_kmeans_stub
        sys.modules["flash_kmeans"] = stub
    if _REF_DIR not in sys.path:
        sys.path.insert(0, _REF_DIR)
    return importlib.import_module("ref_low_bit_fake_quant")
