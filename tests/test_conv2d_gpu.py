"""conv2d (implicit GEMM) on the GPU, through the C ABI, against the oracle and the golden vectors.

Mirrors the reference's tests/test_conv2d.py (x[4,64,16,16], w[512,64,3,3], padding in
{0, (1,1), (0,1), (2,0)}, rtol = atol = 1e-3 against F.conv2d on uniform inputs) and adds
ragged channel counts, odd batch sizes, other filter sizes and strided views.
"""

import numpy as np
import pytest
import torch

from oracle import inputs as oi
from oracle import kernels as ok

from conftest import load_golden
from gpu_util import assert_close, assert_device_healthy, dev, host

pytestmark = pytest.mark.gpu


def run(x, w, padding):
    from ninetoothed_b200 import _capi

    xd, wd = dev(x), dev(w)
    n, _, h, wid = x.shape
    k, _, r, s = w.shape
    y = torch.empty((n, k, h + 2 * padding[0] - r + 1, wid + 2 * padding[1] - s + 1), dtype=xd.dtype, device="cuda")
    _capi.conv2d(xd, wd, y, padding[0], padding[1])
    torch.cuda.synchronize()
    return host(y)


@pytest.mark.parametrize("case", sorted(load_golden("conv2d")))
def test_golden(case):
    g = load_golden("conv2d")[case]
    x, w = oi.conv2d_inputs(tuple(int(v) for v in g["xshape"]), tuple(int(v) for v in g["wshape"]), int(g["seed"]))
    out = run(x, w, tuple(int(v) for v in g["padding"]))
    assert out.shape == g["out"].shape
    assert_close(out, g["out"])
    assert_device_healthy()


@pytest.mark.parametrize("padding", [(0, 0), (1, 1), (0, 1), (2, 0)])
def test_reference_test_shapes(padding):
    """tests/test_conv2d.py:116-133 of the reference: uniform [0,1) inputs, rtol = atol = 1e-3."""
    rng = np.random.default_rng(9)
    x = rng.random((4, 64, 16, 16), dtype=np.float32).astype(np.float16)
    w = rng.random((512, 64, 3, 3), dtype=np.float32).astype(np.float16)
    out = run(x, w, padding)
    expected = torch.nn.functional.conv2d(dev(x), dev(w), padding=padding)
    assert_close(out, host(expected), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("xshape, wshape, padding", [
    ((2, 64, 8, 8), (256, 64, 3, 3), (1, 1)),
    ((1, 16, 5, 7), (8, 16, 3, 3), (1, 1)),       # one image (odd batch), small channel counts
    ((3, 20, 9, 11), (40, 20, 3, 3), (1, 2)),     # channels not a multiple of 8
    ((2, 72, 12, 12), (300, 72, 1, 1), (0, 0)),   # 1x1 filter, K > one tile
    ((2, 32, 12, 10), (64, 32, 5, 3), (2, 1)),    # 5x3 filter
    ((5, 128, 20, 20), (256, 128, 3, 3), (1, 1)),
    # enough tiles for the CTA-pair kernel (4 images per tile): a ragged last pair, and a pair whose second
    # CTA holds no image at all
    ((6, 16, 56, 56), (32, 16, 3, 3), (1, 1)),
    ((5, 24, 50, 60), (40, 24, 3, 3), (1, 0)),
    # the channel tile is 64, 128 or 256 wide by the filter count: both sides of each boundary, single CTAs and pairs
    ((2, 32, 10, 10), (65, 32, 3, 3), (1, 1)),
    ((2, 32, 10, 10), (128, 32, 3, 3), (1, 1)),
    ((2, 32, 10, 10), (129, 32, 3, 3), (1, 1)),
    ((8, 16, 48, 48), (96, 16, 3, 3), (1, 1)),
    ((8, 16, 48, 48), (64, 16, 1, 1), (0, 0)),
    # 1x1 filters without padding on contiguous NCHW tensors run as a batch of GEMMs (no layout pass): several
    # tiles per image on CTA pairs; a channel count that is not a multiple of 64; 7x7 images, whose 49 pixels
    # are not 16-byte rows, stay on the im2col kernel; with padding likewise
    ((4, 256, 28, 28), (512, 256, 1, 1), (0, 0)),
    ((3, 200, 24, 24), (136, 200, 1, 1), (0, 0)),
    ((2, 64, 7, 7), (128, 64, 1, 1), (0, 0)),
    ((2, 64, 8, 8), (128, 64, 1, 1), (1, 1)),
])
def test_shapes(xshape, wshape, padding):
    x, w = oi.conv2d_inputs(xshape, wshape, 90 + xshape[1])
    out = run(x, w, padding)
    assert_close(out, ok.conv2d(x, w, padding, block_m=128, block_n=256, block_k=64))
    assert_device_healthy()


def test_strided_views_and_bf16():
    from ninetoothed_b200 import _capi

    x, w = oi.conv2d_inputs((2, 32, 10, 10), (64, 32, 3, 3), 95)
    expected = ok.conv2d(x, w, (1, 1))
    x_nhwc = dev(x).permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)  # channels-last storage
    y_nhwc = torch.empty(2, 10, 10, 64, dtype=torch.float16, device="cuda").permute(0, 3, 1, 2)
    _capi.conv2d(x_nhwc, dev(w), y_nhwc, 1, 1)
    assert_close(host(y_nhwc), expected)
    xb, wb = dev(x).bfloat16(), dev(w).bfloat16()
    yb = torch.empty(2, 64, 10, 10, dtype=torch.bfloat16, device="cuda")
    _capi.conv2d(xb, wb, yb, 1, 1)
    ref = torch.nn.functional.conv2d(xb.float(), wb.float(), padding=1)
    assert_close(host(yb.float()), host(ref), rtol=2e-2, atol=2e-2)


def test_full_size_linearity_and_sample():
    """x[64,256,56,56] * w[256,256,3,3], padding 1: sampled images against the oracle, and
    homogeneity over the whole output: conv(x, 2w) == 2 conv(x, w) (doubling is exact in fp16
    and fp32, so only outputs in the fp16 subnormal range may differ, by half a subnormal step)."""
    from ninetoothed_b200 import _capi

    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(64, 256, 56, 56, generator=g, device="cuda", dtype=torch.float32).half()
    w = (torch.randn(256, 256, 3, 3, generator=g, device="cuda", dtype=torch.float32) / 48).half()
    y = torch.empty(64, 256, 56, 56, dtype=torch.float16, device="cuda")
    workspace = torch.empty(_capi.conv2d_workspace_size(x, w), dtype=torch.uint8, device="cuda")
    _capi.conv2d(x, w, y, 1, 1, workspace=workspace)
    for n in (0, 63):
        expected = ok.conv2d(host(x[n:n + 1]), host(w), (1, 1), block_m=128, block_n=256, block_k=64)
        assert_close(host(y[n:n + 1]), expected)
    y_double = torch.empty_like(y)
    _capi.conv2d(x, w * 2, y_double, 1, 1, workspace=workspace)
    assert (y_double.float() - 2 * y.float()).abs().max().item() <= 2.0 ** -24
    assert_device_healthy()


def test_rejects_bad_workspace_and_shapes():
    from ninetoothed_b200 import _capi

    x = torch.zeros(2, 16, 8, 8, dtype=torch.float16, device="cuda")
    w = torch.zeros(32, 16, 3, 3, dtype=torch.float16, device="cuda")
    y = torch.zeros(2, 32, 8, 8, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        _capi.conv2d(x, w, y, 1, 1, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))
    with pytest.raises(_capi.KernelLaunchError):
        _capi.conv2d(x, w, y, 0, 0)  # output shape does not match padding 0
    with pytest.raises(_capi.KernelLaunchError):
        _capi.conv2d(x, torch.zeros(32, 8, 3, 3, dtype=torch.float16, device="cuda"), y, 1, 1)


@pytest.mark.parametrize("constexpr_shapes", [False, True])
def test_through_build_like_the_reference_aot_test(constexpr_shapes):
    """tests/test_aot.py:225-301 of the reference with test_build=True: two block-size configurations,
    the call passes sizes, dtype and block sizes after the tensors; rtol = atol = 1e-3 on N(0,1) inputs
    there is for fp32-like error, the fp16 bar is used here."""
    import functools

    import ninetoothed_b200 as ninetoothed
    from examples import definitions as kd

    n, c, h, w, k, r, s = 4, 64, 16, 16, 512, 3, 3
    names = ("n", "c", "h", "w", "k", "r", "s")
    sizes = dict(zip(names, (n, c, h, w, k, r, s))) if constexpr_shapes else dict.fromkeys(names)
    premake = functools.partial(kd.conv2d_premake, **sizes, dtype=ninetoothed.float16)
    configs = (
        ((), {"block_size_m": 64, "block_size_n": 64, "block_size_k": 64}, {}),
        ((), {"block_size_m": 128, "block_size_n": 32, "block_size_k": 64}, {}),
    )
    kernel = ninetoothed.build(premake, configs, caller="cuda", kernel_name="conv2d_build", output_dir="unused")
    x, wt = oi.conv2d_inputs((n, c, h, w), (k, c, r, s), 321)
    y = torch.empty((n, k, h - r + 1, w - s + 1), dtype=torch.float16, device="cuda")
    kernel(dev(x), dev(wt), y, *sizes.values(), ninetoothed.float16, *configs[0][1].values())
    torch.cuda.synchronize()
    assert_close(host(y), ok.conv2d(x, wt, (0, 0), block_m=128, block_n=256, block_k=64))
    assert_device_healthy()


@pytest.mark.parametrize("xshape, wshape, padding", [
    ((4, 64, 16, 16), (512, 64, 3, 3), (1, 1)),     # channels-last x is read in place, y stored 16 bytes at a time
    ((6, 16, 56, 56), (32, 16, 3, 3), (1, 1)),      # ... on the pair kernel
    ((3, 20, 9, 11), (40, 20, 3, 3), (1, 2)),       # channel counts that are not 16-byte rows: the layout pass runs
    ((2, 24, 12, 12), (36, 24, 3, 3), (0, 0)),      # K not a multiple of 8: element-wise stores for the tail chunk
    # 1x1 filters on channels-last tensors are one GEMM over all pixels (bulk tensor stores): ragged in pixels,
    # channels and filters; and a filter count that is not a multiple of 8, which stays on the im2col kernel
    ((3, 200, 25, 24), (136, 200, 1, 1), (0, 0)),
    ((4, 256, 28, 28), (512, 256, 1, 1), (0, 0)),
    ((2, 64, 9, 9), (36, 64, 1, 1), (0, 0)),
])
def test_channels_last_tensors(xshape, wshape, padding):
    from ninetoothed_b200 import _capi

    x, w = oi.conv2d_inputs(xshape, wshape, 400 + xshape[1])
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    n, _, h, wid = xshape
    k, _, r, s = wshape
    y = torch.empty((n, k, h + 2 * padding[0] - r + 1, wid + 2 * padding[1] - s + 1), dtype=torch.float16,
                    device="cuda").contiguous(memory_format=torch.channels_last)
    assert xd.stride(1) == 1 and y.stride(1) == 1
    _capi.conv2d(xd, dev(w), y, padding[0], padding[1])
    torch.cuda.synchronize()
    assert_close(host(y), ok.conv2d(x, w, padding, block_m=128, block_n=256, block_k=64))
    assert_device_healthy()


@pytest.mark.parametrize("channels_last", [False, True])
def test_1x1_filters_seeded_shapes(channels_last):
    """Twelve seeded shapes through the two GEMM paths of 1x1 filters (batched over images for NCHW, one GEMM over
    all pixels for channels-last): image sizes that are and are not multiples of the 64-pixel box, channel and
    filter counts on both sides of the 64-channel K-block and of the 128/256-row tiles, fp16 and bf16."""
    from ninetoothed_b200 import _capi

    rng = np.random.default_rng(20 + channels_last)
    for case in range(12):
        n = int(rng.integers(1, 5))
        c = 8 * int(rng.integers(1, 34))
        k = 8 * int(rng.integers(1, 40))
        h, w = int(rng.integers(1, 5)) * 4, int(rng.integers(1, 9)) * 2 + (0 if not channels_last else int(rng.integers(0, 2)))
        x, f = oi.conv2d_inputs((n, c, h, w), (k, c, 1, 1), 700 + case)
        expected = ok.conv2d(x, f, (0, 0), block_m=128, block_n=256, block_k=64)
        dtype = torch.bfloat16 if case % 3 == 2 else torch.float16
        xd, fd = dev(x).to(dtype), dev(f).to(dtype)
        y = torch.full((n, k, h, w), float("nan"), dtype=dtype, device="cuda")
        if channels_last:
            xd, y = xd.contiguous(memory_format=torch.channels_last), y.contiguous(memory_format=torch.channels_last)
        _capi.conv2d(xd, fd, y, 0, 0)
        torch.cuda.synchronize()
        if dtype == torch.bfloat16:
            # (the oracle's inputs are fp16; the bf16 case is checked against the fp32 product of the rounded inputs)
            rounded = torch.nn.functional.conv2d(xd.float().contiguous(), fd.float())
            assert_close(host(y.float()), host(rounded), rtol=2e-2, atol=2e-2)
        else:
            assert_close(host(y), expected)
    assert_device_healthy()


@pytest.mark.parametrize("xshape, wshape, padding", [
    ((4, 64, 16, 16), (512, 64, 3, 3), (1, 1)),
    ((3, 40, 9, 11), (72, 40, 5, 3), (2, 1)),      # channels not a multiple of 64: zeros are read beyond them
    ((6, 16, 56, 56), (32, 16, 3, 3), (1, 1)),      # the pair kernel
    ((2, 20, 9, 9), (40, 20, 3, 3), (1, 1)),        # 20 channels are not 16-byte rows: the filter is re-laid-out
])
def test_channels_last_filter_is_read_in_place(xshape, wshape, padding):
    """A channels-last filter (what torch gives the weights of a channels-last model) needs no re-layout pass:
    with a channels-last input the whole convolution is then a single launch."""
    from ninetoothed_b200 import _capi

    x, w = oi.conv2d_inputs(xshape, wshape, 500 + xshape[1])
    xd = dev(x).contiguous(memory_format=torch.channels_last)
    wd = dev(w).contiguous(memory_format=torch.channels_last)
    n, _, h, wid = xshape
    k, _, r, s = wshape
    y = torch.empty((n, k, h + 2 * padding[0] - r + 1, wid + 2 * padding[1] - s + 1), dtype=torch.float16,
                    device="cuda").contiguous(memory_format=torch.channels_last)
    assert wd.stride(1) == 1
    _capi.conv2d(xd, wd, y, padding[0], padding[1])
    torch.cuda.synchronize()
    assert_close(host(y), ok.conv2d(x, w, padding, block_m=128, block_n=256, block_k=64))
    # and with an NCHW input, whose layout pass then runs alone
    y2 = torch.empty_like(y, memory_format=torch.contiguous_format)
    _capi.conv2d(dev(x), wd, y2, padding[0], padding[1])
    assert_close(host(y2), host(y), rtol=0, atol=0)
    assert_device_healthy()
