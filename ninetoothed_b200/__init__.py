"""B200-native kernels behind the NineToothed operator API.

``make`` / ``jit`` / ``build`` / ``Tensor`` / ``Symbol`` / ``block_size`` and the dtype tags
mirror the reference's package surface (``src/ninetoothed/__init__.py`` in the
reference project) for the arrangements this library implements by hand:
matmul, addmm, row softmax, fused attention and conv2d.  The kernels are CUDA for
sm_100a in ``libninetoothed_b200.so`` (C ABI: ``include/ninetoothed_b200.h``).
"""

from ninetoothed_b200.dtype import (
    bfloat16,
    float16,
    float32,
    float64,
    int8,
    int16,
    int32,
    int64,
    uint8,
    uint16,
    uint32,
    uint64,
)
from ninetoothed_b200.dispatch import build
from ninetoothed_b200.make import jit, make
from ninetoothed_b200.recognition import UnsupportedKernelError
from ninetoothed_b200.symbol import Symbol, block_size
from ninetoothed_b200.tensor import Tensor

__all__ = [
    "Symbol", "Tensor", "UnsupportedKernelError", "bfloat16", "block_size", "build", "float16", "float32", "float64", "int8",
    "int16", "int32", "int64", "jit", "make", "uint8", "uint16", "uint32", "uint64",
]
