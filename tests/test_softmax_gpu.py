"""Row softmax on the GPU, through the C ABI, against the oracle and the golden vectors.

Mirrors the reference's tests/test_softmax.py (1823 x 781 fp32, allclose) and adds
the fp16 storage / fp32 math configuration with 4*N(0,1) inputs.
Tolerances: fp32 output rtol 1e-5 / atol 1e-7 (the reference test's allclose);
fp16 output rtol 1e-2 / atol 1e-2; every row sums to 1 within 1e-3.
"""

import numpy as np
import pytest
import torch

from oracle import inputs as oi
from oracle import kernels as ok

from conftest import load_golden
from gpu_util import assert_close, assert_device_healthy, dev, host

pytestmark = pytest.mark.gpu


def run(x):
    from ninetoothed_b200 import _capi

    xd = dev(x)
    yd = torch.empty_like(xd)
    _capi.softmax(xd, yd)
    torch.cuda.synchronize()
    return host(yd)


@pytest.mark.parametrize("case", sorted(load_golden("softmax")))
def test_golden(case):
    g = load_golden("softmax")[case]
    rows, cols = (int(v) for v in g["shape"])
    if case.startswith("fp32"):
        x = oi.softmax_inputs(rows, cols, int(g["seed"]), dtype=np.float32)
        np.testing.assert_allclose(run(x), g["out"], rtol=1e-5, atol=1e-7)
    else:
        x = oi.softmax_inputs(rows, cols, int(g["seed"]), scale=float(g["scale"]))
        assert_close(run(x), g["out"])


def test_reference_test_shape_fp32():
    """tests/test_softmax.py:30-40 of the reference: 1823 x 781, uniform inputs, fp32."""
    rng = np.random.default_rng(5)
    x = rng.random((1823, 781), dtype=np.float32)
    y = run(x)
    np.testing.assert_allclose(y, ok.softmax(x), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("rows, cols", [(1, 8), (3, 8192), (257, 1024), (64, 4096), (5, 16384), (2, 65536),
                                        (7, 1000), (4, 8200), (1, 1), (33, 129),
                                        # rows staged in shared memory: long ones, and column counts that leave
                                        # every row at another offset within a 16-byte vector
                                        (6, 32768), (3, 50257), (9, 781), (5, 7), (4, 100003), (2, 120000)])
def test_shapes_fp16(rows, cols):
    x = oi.softmax_inputs(rows, cols, 100 + cols, scale=4.0)
    y = run(x)
    assert_close(y, ok.softmax(x))
    assert np.abs(y.astype(np.float64).sum(-1) - 1).max() < 1e-3


def test_bf16_and_strided():
    from ninetoothed_b200 import _capi

    x = torch.from_numpy(oi.softmax_inputs(64, 2048, 7, dtype=np.float32, scale=4.0)).cuda()
    xb = x.to(torch.bfloat16)
    yb = torch.empty_like(xb)
    _capi.softmax(xb, yb)
    expected = ok.softmax(host(xb.float()))
    assert_close(host(yb.float()), expected, rtol=2e-2, atol=1e-2)
    # a column-sliced (row stride > cols) fp16 view and a transposed view
    xh = x.to(torch.float16)
    wide = torch.zeros(64, 4096, dtype=torch.float16, device="cuda")
    wide[:, :2048] = xh
    out = torch.empty(64, 4096, dtype=torch.float16, device="cuda")
    _capi.softmax(wide[:, :2048], out[:, :2048])
    assert_close(host(out[:, :2048]), ok.softmax(host(xh)))
    xt = xh.t()  # [2048, 64], inner stride 2048
    yt = torch.empty(2048, 64, dtype=torch.float16, device="cuda")
    _capi.softmax(xt, yt)
    assert_close(host(yt), ok.softmax(host(xt.contiguous())))
    assert_device_healthy()


def test_rows_whose_input_and_output_sit_at_different_offsets():
    """Odd column count, and an output view that starts 3 elements into its buffer: the staged kernel's
    element-wise store path."""
    from ninetoothed_b200 import _capi

    x = dev(oi.softmax_inputs(12, 999, 8, scale=4.0))
    buffer = torch.zeros(12 * 999 + 3, dtype=torch.float16, device="cuda")
    y = buffer[3:].view(12, 999)
    _capi.softmax(x, y)
    torch.cuda.synchronize()
    assert_close(host(y), ok.softmax(host(x)))
    assert float(buffer[:3].abs().sum()) == 0.0
    x32 = dev(oi.softmax_inputs(5, 1001, 9, dtype=np.float32, scale=4.0))
    y32 = torch.empty_like(x32)
    _capi.softmax(x32, y32)
    assert_close(host(y32), ok.softmax(host(x32)), rtol=1e-5, atol=1e-6)
    assert_device_healthy()


def test_full_size_rows_sum_to_one():
    """The benchmark configuration: X[65536, 8192] fp16 = 4*N(0,1)."""
    g = torch.Generator(device="cuda").manual_seed(2)
    x = (4 * torch.randn(65536, 8192, generator=g, device="cuda", dtype=torch.float32)).to(torch.float16)
    from ninetoothed_b200 import _capi

    y = torch.empty_like(x)
    _capi.softmax(x, y)
    sums = y.float().sum(-1)
    assert (sums - 1).abs().max().item() < 1e-3
    # softmax is shift-invariant and preserves order within a row
    sample = slice(0, 64)
    assert_close(host(y[sample]), ok.softmax(host(x[sample])))
    assert torch.equal(y[sample].argmax(-1), x[sample].argmax(-1))


def test_rejects_mismatched_shapes():
    from ninetoothed_b200 import _capi

    x = torch.zeros(4, 8, dtype=torch.float16, device="cuda")
    y = torch.zeros(4, 16, dtype=torch.float16, device="cuda")
    with pytest.raises(_capi.KernelLaunchError):
        _capi.softmax(x, y)
