"""Stages the reference project's Python package for runs on a GPU machine.

TEST INFRASTRUCTURE ONLY: nothing the library ships imports what this stages.

The reference (DongyunZou/low-bit-attention-fake-quant) is pure Python + Triton:
nothing of it compiles, but its kernels only run on a GPU. This script copies
its package ``src/low_bit_fake_quant`` (as it lies in a checkout of the
reference, unmodified) to ``oracle/_ref/ref_low_bit_fake_quant`` -- a folder
that version control ignores, so the reference's sources never enter this
repository's history, but that travels with the working tree to a GPU machine.
The copy is renamed because this repository's own package carries the
reference's name (it is a drop-in); the reference uses relative imports
throughout, so the renamed copy imports unchanged. ``oracle/ref_gpu.py`` loads
it; ``tests/golden/make_golden_gpu.py`` runs it to record golden vectors.

    python oracle/make_ref.py /path/to/reference

Without a reference checkout at the given path this is a no-op (exit 0).
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "ref_low_bit_fake_quant")


def stage(reference_root: str) -> bool:
    src = os.path.join(reference_root, "src", "low_bit_fake_quant")
    if not os.path.isdir(src):
        print(f"make_ref: no reference package at {src}; nothing staged")
        return False
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(os.path.dirname(DEST), exist_ok=True)
    shutil.copytree(src, DEST, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    print(f"make_ref: staged {src} -> {DEST}")
    return True


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_ref.py /path/to/reference")
    stage(sys.argv[1])
