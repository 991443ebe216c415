"""conv2d on the library's built-in scratch array (launch_conv2d_static_workspace).

Some users of this library cannot allocate device memory for the conv2d workspace: a
C host that was only handed tensors and a stream, a plugin inside a framework whose
allocator owns the whole GPU, a service with a memory budget fixed at start-up.  This
entry point serves them from an array that ships inside the library.  The test calls
it through the C ABI twice in a row, with different problems so that the second call
finds the first one's leftovers in the array, and checks each result against the
ordinary entry point (launch_conv2d with a caller-provided workspace) and against the
numpy oracle, within the tolerance of the other conv2d tests (rtol 1e-2 / atol 1e-2).

Collected last on purpose: a run that stops at the first failure has then already
run every other test.
"""

import pytest
import torch

from oracle import inputs as oi
from oracle import kernels as ok

from gpu_util import assert_close, assert_device_healthy, dev, host

pytestmark = pytest.mark.gpu


def both_ways(xshape, wshape, padding, seed):
    from ninetoothed_b200 import _capi

    x_host, w_host = oi.conv2d_inputs(xshape, wshape, seed)
    x, w = dev(x_host), dev(w_host)
    n, _, h, wid = xshape
    k, _, r, s = wshape
    yshape = (n, k, h + 2 * padding[0] - r + 1, wid + 2 * padding[1] - s + 1)
    expected = torch.empty(yshape, dtype=torch.float16, device="cuda")
    _capi.conv2d(x, w, expected, padding[0], padding[1])  # existing entry point, torch-allocated workspace
    actual = torch.full(yshape, float("nan"), dtype=torch.float16, device="cuda")
    free_before = torch.cuda.mem_get_info()[0]
    reserved_before = torch.cuda.memory_reserved()
    _capi.conv2d_static_workspace(x, w, actual, padding[0], padding[1])
    torch.cuda.synchronize()
    assert_close(host(actual), ok.conv2d(x_host, w_host, padding, block_m=64, block_n=64, block_k=64))  # the oracle
    return actual, expected, free_before - torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved() - reserved_before


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    from ninetoothed_b200 import _capi

    # first call: 72 channels (padded to 72), ~5.6 MB of scratch
    actual, expected, _, _ = both_ways((6, 72, 40, 40), (96, 72, 3, 3), (1, 1), 301)
    assert_close(host(actual), host(expected))
    # second call: other shape, fewer channels, different padding: the array still holds the first call's data
    actual, expected, device_growth, torch_growth = both_ways((3, 20, 33, 29), (40, 20, 5, 3), (2, 0), 302)
    assert_close(host(actual), host(expected))
    assert torch.equal(actual, expected)  # same kernels, same arithmetic
    # the set-up happened in the first call; the second one must not have taken device memory
    assert torch_growth == 0
    assert device_growth < (1 << 20)
    assert _capi.conv2d_workspace_size(dev(oi.normal(1, (3, 20, 33, 29))), dev(oi.normal(2, (40, 20, 5, 3)))) > (1 << 16)
    assert_device_healthy()


def test_problems_beyond_the_built_in_array_are_rejected():
    from ninetoothed_b200 import _capi

    x = torch.zeros(24, 256, 56, 56, dtype=torch.float16, device="cuda")  # needs ~38.6 MB of scratch
    w = torch.zeros(64, 256, 3, 3, dtype=torch.float16, device="cuda")
    y = torch.zeros(24, 64, 56, 56, dtype=torch.float16, device="cuda")
    assert _capi.conv2d_workspace_size(x, w) > _capi.STATIC_WORKSPACE_BYTES
    with pytest.raises(_capi.KernelLaunchError, match="built-in array holds"):
        _capi.conv2d_static_workspace(x, w, y, 1, 1)


def test_only_what_a_launch_touches_counts_against_the_limit():
    """The same oversized problem on channels-last tensors reads input and filter in place and writes no scratch,
    and an unpadded 1 x 1 filter never touches any: both are served, and agree with the ordinary entry point."""
    from ninetoothed_b200 import _capi

    x_host, w_host = oi.conv2d_inputs((24, 256, 56, 56), (64, 256, 3, 3), 303)
    x = dev(x_host).contiguous(memory_format=torch.channels_last)
    w = dev(w_host).contiguous(memory_format=torch.channels_last)
    assert _capi.conv2d_workspace_size(x, w) > _capi.STATIC_WORKSPACE_BYTES
    y = torch.empty(24, 64, 56, 56, dtype=torch.float16, device="cuda").contiguous(memory_format=torch.channels_last)
    expected = torch.empty_like(y)
    _capi.conv2d(x, w, expected, 1, 1)
    _capi.conv2d_static_workspace(x, w, y, 1, 1)
    assert torch.equal(y, expected)
    image = ok.conv2d(x_host[:1], w_host, (1, 1), block_m=64, block_n=64, block_k=64)  # one image against the oracle
    assert_close(host(y[:1]), image)

    x1_host, w1_host = oi.conv2d_inputs((48, 256, 56, 56), (128, 256, 1, 1), 304)  # 77 MB of nominal scratch
    x1, w1 = dev(x1_host), dev(w1_host)
    assert _capi.conv2d_workspace_size(x1, w1) > _capi.STATIC_WORKSPACE_BYTES
    y1 = torch.empty(48, 128, 56, 56, dtype=torch.float16, device="cuda")
    expected1 = torch.empty_like(y1)
    _capi.conv2d(x1, w1, expected1, 0, 0)
    _capi.conv2d_static_workspace(x1, w1, y1, 0, 0)
    assert torch.equal(y1, expected1)
    assert_close(host(y1[:1]), ok.conv2d(x1_host[:1], w1_host, (0, 0), block_m=64, block_n=64, block_k=64))
    assert_device_healthy()
