"""max_pool2d on the GPU, through the front door and the C ABI, against the oracle and the golden vectors.

Mirrors the reference's tests/test_max_pool2d.py (x[32,3,64,64] fp16, 3 x 3 windows, floor and ceil
mode, torch.allclose against F.max_pool2d) and adds other windows, ragged widths, strided views and
the other data types.  max is exact, so every comparison is bit for bit.
"""

import numpy as np
import pytest
import torch

from oracle import kernels as ok

from conftest import load_golden
from gpu_util import assert_device_healthy, dev, host

pytestmark = pytest.mark.gpu


def output_shape(shape, window, ceil_mode):
    n, c, h, w = shape
    r, s = window
    div = (lambda a, b: -(-a // b)) if ceil_mode else (lambda a, b: a // b)
    return (n, c, div(h - r, r) + 1, div(w - s, s) + 1)


def run(x, window, ceil_mode):
    from examples import definitions as kd

    xd = x if isinstance(x, torch.Tensor) else dev(x)
    y = torch.empty(output_shape(tuple(xd.shape), window, ceil_mode), dtype=xd.dtype, device="cuda")
    kd.make_max_pool2d(ceil_mode)(xd, y, WINDOW_HEIGHT=window[0], WINDOW_WIDTH=window[1])
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("case", sorted(load_golden("max_pool2d")))
def test_golden(case):
    g = load_golden("max_pool2d")[case]
    x = ok.normal(int(g["seed"]), tuple(int(v) for v in g["shape"]), np.float16)
    out = run(x, tuple(int(v) for v in g["window"]), bool(g["ceil_mode"]))
    assert np.array_equal(host(out), g["out"])
    assert_device_healthy()


@pytest.mark.parametrize("ceil_mode", [False, True])
def test_reference_test_shape(ceil_mode):
    """tests/test_max_pool2d.py:66-83 of the reference."""
    x = ok.normal(40, (32, 3, 64, 64), np.float16)
    out = run(x, (3, 3), ceil_mode)
    expected = torch.nn.functional.max_pool2d(dev(x), (3, 3), ceil_mode=ceil_mode)
    assert torch.equal(out, expected)
    assert np.array_equal(host(out), ok.max_pool2d(x, (3, 3), ceil_mode))


@pytest.mark.parametrize("ceil_mode", [False, True])
@pytest.mark.parametrize("shape, window", [
    ((2, 5, 56, 56), (2, 2)),     # whole rows go through the 16-byte path
    ((1, 3, 17, 41), (2, 2)),     # rows that are not 16-byte addressable
    ((2, 2, 33, 72), (3, 4)),     # four-wide windows, ragged height
    ((1, 4, 40, 130), (1, 1)),    # the identity
    ((1, 2, 64, 96), (5, 6)),     # windows wider than the 16-byte path takes
    ((3, 1, 16, 16), (16, 16)),   # one window per plane (the largest the reference's symbols allow)
])
def test_shapes(shape, window, ceil_mode):
    x = ok.normal(41 + shape[3], shape, np.float16)
    out = run(x, window, ceil_mode)
    assert np.array_equal(host(out), ok.max_pool2d(x, window, ceil_mode))
    assert_device_healthy()


def test_other_dtypes_and_strided_views():
    from ninetoothed_b200 import _capi

    rng = np.random.default_rng(5)
    x32 = rng.standard_normal((2, 3, 24, 40)).astype(np.float32)
    assert np.array_equal(host(run(x32, (2, 2), False)), ok.max_pool2d(x32, (2, 2), False))
    xb = torch.from_numpy(x32).cuda().bfloat16()
    expected = torch.nn.functional.max_pool2d(xb.float(), (3, 2), ceil_mode=True).bfloat16()
    assert torch.equal(run(xb, (3, 2), True), expected)
    # a channels-last view and an output that is a slice of a larger buffer
    xh = torch.from_numpy(x32).cuda().half().permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)
    assert xh.stride(3) != 1
    big = torch.zeros(2, 3, 12, 64, dtype=torch.float16, device="cuda")
    view = big[:, :, :, 3:23]
    _capi.max_pool2d(xh, view, 2, 2, False)
    torch.cuda.synchronize()
    assert torch.equal(view, torch.nn.functional.max_pool2d(xh.contiguous(), (2, 2)))
    assert float(big[:, :, :, :3].abs().sum()) == 0.0 and float(big[:, :, :, 23:].abs().sum()) == 0.0
    assert_device_healthy()


def test_full_size_properties():
    """At the benchmark's size: pooling 2 x 2 twice equals pooling 4 x 4 once (max is associative), a
    1 x 1 window is the identity, and every output is one of its window's inputs (checked on a sample)."""
    gen = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(64, 256, 112, 112, dtype=torch.float16, device="cuda", generator=gen)
    once = run(x, (4, 4), False)
    twice = run(run(x, (2, 2), False), (2, 2), False)
    assert torch.equal(once, twice)
    assert torch.equal(run(x[:4], (1, 1), False), x[:4])
    sample = x[5, 17].float().cpu().numpy()[None, None]
    assert np.array_equal(host(run(x[5:6, 17:18], (2, 2), True)).astype(np.float32), ok.max_pool2d(sample, (2, 2), True))
    assert_device_healthy()


def test_rejects_bad_arguments():
    from ninetoothed_b200 import _capi

    x = torch.zeros(1, 1, 8, 8, dtype=torch.float16, device="cuda")
    with pytest.raises(_capi.KernelLaunchError):   # floor-mode output shape for a ceil-mode call
        _capi.max_pool2d(x, torch.zeros(1, 1, 2, 2, dtype=torch.float16, device="cuda"), 3, 3, True)
    with pytest.raises(_capi.KernelLaunchError):   # window larger than the input
        _capi.max_pool2d(x, torch.zeros(1, 1, 1, 1, dtype=torch.float16, device="cuda"), 9, 2, False)
    with pytest.raises(_capi.KernelLaunchError):
        _capi.max_pool2d(x.double(), torch.zeros(1, 1, 4, 4, dtype=torch.float64, device="cuda"), 2, 2, False)
