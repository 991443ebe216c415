"""Seeded input recipes shared by the golden generator, the tests and bench.

TEST INFRASTRUCTURE ONLY.  Each recipe returns numpy arrays drawn from
``oracle.kernels.normal``; ``checksum`` is what the golden files store so a
drifting generator is detected instead of silently comparing different inputs.
"""

import hashlib

import numpy as np

from oracle.kernels import normal


def checksum(*arrays):
    digest = hashlib.sha256()
    for a in arrays:
        digest.update(np.ascontiguousarray(a).tobytes())
    return digest.hexdigest()


def matmul_inputs(m, n, k, seed, dtype=np.float16):
    return normal(seed, (m, k), dtype), normal(seed + 1000, (k, n), dtype)


def addmm_inputs(m, n, k, seed, dtype=np.float16):
    return (
        normal(seed, (m, n), dtype),
        normal(seed + 1000, (m, k), dtype),
        normal(seed + 2000, (k, n), dtype),
    )


def softmax_inputs(rows, cols, seed, dtype=np.float16, scale=1.0):
    return normal(seed, (rows, cols), dtype, scale=scale)


def attention_inputs(shape, seed, dtype=np.float16):
    return (
        normal(seed, shape, dtype),
        normal(seed + 1000, shape, dtype),
        normal(seed + 2000, shape, dtype),
    )


def conv2d_inputs(xshape, wshape, seed, dtype=np.float16):
    fan_in = wshape[1] * wshape[2] * wshape[3]
    return normal(seed, xshape, dtype), normal(seed + 1000, wshape, dtype, scale=1.0 / np.sqrt(fan_in))
