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


def e5m2_from_fp16(x):
    """fp16 -> 8-bit e5m2 bytes, round to nearest even: e5m2 is the high byte of the fp16 encoding, so the
    low byte is rounded away (what ``tensor.to(torch.float8_e5m2)`` does for finite values in range)."""
    bits = np.ascontiguousarray(x, dtype=np.float16).view(np.uint16).astype(np.uint32)
    keep_odd = (bits >> 8) & 1
    return ((bits + 0x7F + keep_odd) >> 8).astype(np.uint8)


def e5m2_to_fp16(b):
    """8-bit e5m2 bytes -> the fp16 with the same value (exact)."""
    return (np.ascontiguousarray(b, dtype=np.uint8).astype(np.uint16) << 8).view(np.float16)


def matmul_e5m2_inputs(m, n, k, seed):
    """Operands of the reference's 8-bit matmul test (tests/test_matmul.py:72-80): N(0,1) drawn in fp16 and
    rounded to e5m2.  Returns lhs [M, K] and rhs stored as [N, K] (its transpose is the [K, N] operand, so
    K is the unit-stride dimension of both, as in the test)."""
    a, b = matmul_inputs(m, n, k, seed)
    return e5m2_from_fp16(a), np.ascontiguousarray(e5m2_from_fp16(b).T)
