"""CPU oracle for the block-FP8 W8A8 linear + fused-MoE path.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this
directory: it is the checker used by the parity tests, by the smoke check and
by the CPU-baseline leg of the benchmark, never the thing measured or shipped.

Parity status: PINNED. Every function in ``oracle.block_fp8`` is compared
bit-for-bit (integer / byte outputs) or to float equality with the reference's
own torch-native functions in ``tests/golden/make_golden.py`` (run where the
reference tree is importable); the resulting vectors are committed under
``tests/golden/`` and re-checked by the CPU test-suite. One deliberate difference: where
the reference calls ``torch.topk(..., sorted=False)`` (order of the k results and ties
unspecified) the routing functions here return descending order with the lower index first
on ties, the rule of the reference's CUDA routing kernels; those vectors are compared by
expert id.

Evaluate it on CPU tensors. The functions run on CUDA tensors too, but there torch divides by a
Python scalar through its reciprocal (``amax / 448`` becomes ``amax * (1/448)``), which is not
the arithmetic restated here and moves FP8 ties.
"""
from .block_fp8 import *  # noqa: F401,F403
