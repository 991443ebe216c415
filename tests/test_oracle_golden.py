"""Pins the numpy oracle against outputs of the reference itself.

The vectors under tests/golden/ were produced by the reference's own kernels
(its test-suite definitions of matmul, addmm, softmax, attention and conv2d,
tests/test_{matmul,addmm,softmax,attention,conv2d}.py in the reference project)
run on CPU through Triton's interpreter; see tests/golden/generate.py.
"""

import numpy as np
import pytest

from oracle import inputs as oi
from oracle import kernels as ok

from conftest import load_golden


def ulp_fp16(a, b):
    """Largest distance, in fp16 units in the last place, between two fp16 arrays."""
    ai = a.astype(np.float16).view(np.int16).astype(np.int32)
    bi = b.astype(np.float16).view(np.int16).astype(np.int32)
    ai = np.where(ai < 0, -32768 - ai, ai)
    bi = np.where(bi < 0, -32768 - bi, bi)
    return int(np.abs(ai - bi).max())


@pytest.mark.parametrize("case", sorted(load_golden("matmul")))
def test_matmul(case):
    g = load_golden("matmul")[case]
    m, n, k = (int(v) for v in g["shape"])
    a, b = oi.matmul_inputs(m, n, k, int(g["seed"]))
    assert oi.checksum(a, b) == str(g["inputs"])
    out = ok.matmul(a, b, np.float16, *(int(v) for v in g["blocks"]))
    # Same blocks, same order, fp32 accumulate: only the order of adds inside one
    # BLAS call may differ, so almost every element is bit-identical.
    assert ulp_fp16(out, g["out"]) <= 1
    assert (out == g["out"]).mean() > 0.999


@pytest.mark.parametrize("case", ["square", "ragged"])
def test_bmm(case):
    g = load_golden("bmm")[case]
    batch, m, n, k = (int(v) for v in g["shape"])
    seed = int(g["seed"])
    a, b = ok.normal(seed, (batch, m, k), np.float16), ok.normal(seed + 1000, (batch, k, n), np.float16)
    assert oi.checksum(a, b) == str(g["inputs"])
    out = ok.bmm(a, b, np.float16, *(int(v) for v in g["blocks"]))
    assert ulp_fp16(out, g["out"]) <= 1
    assert (out == g["out"]).mean() > 0.999


@pytest.mark.parametrize("case", sorted(load_golden("addmm")))
def test_addmm(case):
    g = load_golden("addmm")[case]
    m, n, k = (int(v) for v in g["shape"])
    c, a, b = oi.addmm_inputs(m, n, k, int(g["seed"]))
    assert oi.checksum(c, a, b) == str(g["inputs"])
    out = ok.addmm(c, a, b, float(g["beta"]), float(g["alpha"]), np.float16, *(int(v) for v in g["blocks"]))
    assert ulp_fp16(out, g["out"]) <= 1
    assert (out == g["out"]).mean() > 0.999


def test_addmm_rounds_product_to_fp16_before_epilogue():
    """The double rounding is observable: skipping it changes golden elements."""
    g = load_golden("addmm")["scaled_ragged"]
    m, n, k = (int(v) for v in g["shape"])
    c, a, b = oi.addmm_inputs(m, n, k, int(g["seed"]))
    acc = ok.matmul_acc(a, b, *(int(v) for v in g["blocks"]))
    single = (np.float32(g["beta"]) * c.astype(np.float32) + np.float32(g["alpha"]) * acc).astype(np.float16)
    double = ok.addmm(c, a, b, float(g["beta"]), float(g["alpha"]), np.float16, *(int(v) for v in g["blocks"]))
    assert (double == g["out"]).mean() > (single == g["out"]).mean()


@pytest.mark.parametrize("case", sorted(load_golden("softmax")))
def test_softmax(case):
    g = load_golden("softmax")[case]
    rows, cols = (int(v) for v in g["shape"])
    if case.startswith("fp32"):
        x = oi.softmax_inputs(rows, cols, int(g["seed"]), dtype=np.float32)
        out = ok.softmax(x)
        assert oi.checksum(x) == str(g["inputs"])
        np.testing.assert_allclose(out, g["out"], rtol=1e-6, atol=1e-9)
    else:
        x = oi.softmax_inputs(rows, cols, int(g["seed"]), scale=float(g["scale"]))
        assert oi.checksum(x) == str(g["inputs"])
        out = ok.softmax(x)
        assert ulp_fp16(out, g["out"]) <= 1
    assert np.abs(out.astype(np.float64).sum(-1) - 1).max() < 1e-3


@pytest.mark.parametrize("case", sorted(load_golden("attention")))
def test_attention(case):
    g = load_golden("attention")[case]
    shape = tuple(int(v) for v in g["shape"])
    q, k, v = oi.attention_inputs(shape, int(g["seed"]))
    assert oi.checksum(q, k, v) == str(g["inputs"])
    scale = float(g["scale"])
    out = ok.attention(q, k, v, bool(g["is_causal"]), int(g["blocks"][0]), int(g["blocks"][1]),
                       scale=None if scale < 0 else scale)
    assert ulp_fp16(out, g["out"]) <= 2
    assert (out == g["out"]).mean() > 0.99


@pytest.mark.parametrize("case", sorted(load_golden("conv2d")))
def test_conv2d(case):
    g = load_golden("conv2d")[case]
    xshape = tuple(int(v) for v in g["xshape"])
    wshape = tuple(int(v) for v in g["wshape"])
    x, w = oi.conv2d_inputs(xshape, wshape, int(g["seed"]))
    assert oi.checksum(x, w) == str(g["inputs"])
    out = ok.conv2d(x, w, tuple(int(v) for v in g["padding"]), np.float16, *(int(v) for v in g["blocks"]))
    assert out.shape == g["out"].shape
    assert ulp_fp16(out, g["out"]) <= 1
    assert (out == g["out"]).mean() > 0.999


@pytest.mark.parametrize("case", sorted(load_golden("max_pool2d")))
def test_max_pool2d_matches_reference_output(case):
    """max is exact: the oracle must reproduce the reference's bits."""
    g = load_golden("max_pool2d")[case]
    x = ok.normal(int(g["seed"]), tuple(int(v) for v in g["shape"]), np.float16)
    assert oi.checksum(x) == g["inputs"]
    out = ok.max_pool2d(x, tuple(int(v) for v in g["window"]), bool(g["ceil_mode"]))
    assert out.dtype == g["out"].dtype and np.array_equal(out, g["out"])


@pytest.mark.parametrize("case", sorted(load_golden("matmul_e5m2")))
def test_matmul_e5m2(case):
    """8-bit e5m2 operands are exact fp16 values: the fp16 oracle on the decoded operands is the oracle."""
    g = load_golden("matmul_e5m2")[case]
    m, n, k = (int(v) for v in g["shape"])
    a8, bt8 = oi.matmul_e5m2_inputs(m, n, k, int(g["seed"]))
    assert oi.checksum(a8, bt8) == str(g["inputs"])
    out = ok.matmul(oi.e5m2_to_fp16(a8), oi.e5m2_to_fp16(bt8).T, np.float16, *(int(v) for v in g["blocks"]))
    assert ulp_fp16(out, g["out"]) <= 1
    assert (out == g["out"]).mean() > 0.999


def test_e5m2_rounding_is_nearest_even():
    x = np.array([1.0, 1.125, 1.375, 1.25, -3.0, 0.0, 6.1e-5], dtype=np.float16)
    # 1.125 is halfway between 1.0 and 1.25 -> even (1.0); 1.375 is halfway between 1.25 and 1.5 -> even (1.5)
    back = oi.e5m2_to_fp16(oi.e5m2_from_fp16(x))
    assert back.tolist()[:5] == [1.0, 1.0, 1.5, 1.25, -3.0] and back[5] == 0.0
