"""CPU oracle of the fake-quant attention path: TEST INFRASTRUCTURE ONLY.

A plain-torch restatement of the reference algorithms (``quant_ops``: the
quantizers, smoothing and Hadamard kernels; ``k12``: the streaming attention
kernel; ``api``: the orchestration and k-means reorder). Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import it, as the checker or the timed CPU baseline -- never the shipped path.
"""
