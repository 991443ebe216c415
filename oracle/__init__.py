"""CPU oracle for the four NineToothed hot-path kernels.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is the checker used by ``tests/``, by the smoke entry point and
by the CPU-baseline leg of ``bench.py``.  The product path is the CUDA library
and fails loudly when that library is missing.

``oracle.kernels`` restates, in numpy, the arithmetic of the kernels that the
reference's arrange-and-apply definitions produce (matmul, addmm, row softmax,
fused attention with online softmax, conv2d as implicit GEMM), block by block
and rounding point by rounding point.  The restatement is pinned against
outputs of the reference itself, executed on CPU through Triton's interpreter
by ``tests/golden/generate.py``; the resulting vectors are committed under
``tests/golden/`` and replayed by ``tests/test_oracle_golden.py``.
"""
