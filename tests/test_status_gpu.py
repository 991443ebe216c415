"""The device status word, the bounded-wait give-up path, and the notes about slow paths.

A wait that runs out must not hang or fault anything: the library's self-test kernel waits a few
microseconds on a barrier nobody arrives at, gives up, records its code and returns; the host reads
NINETOOTHED_B200_ERR_TIMEOUT with the code, a second read finds the word cleared, and the context
runs the next kernel as if nothing had happened.
"""

import warnings

import numpy as np
import pytest
import torch

from oracle import inputs as oi
from oracle import kernels as ok

from gpu_util import assert_close, assert_device_healthy, dev, host

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    from ninetoothed_b200 import _capi

    assert _capi.device_status(clear=True) == 0
    _capi.selftest_wait_timeout(limit_ns=5000)
    result, word = _capi.device_status_result(clear=False)
    assert result == _capi.ERR_TIMEOUT
    assert word == 0x10000000 | (15 << 16) | 0x5E1F  # STATUS_WAIT_TIMEOUT | self-test kernel id | its wait code
    assert "wait gave up" in _capi.library().ninetoothed_b200_last_error().decode()
    assert _capi.device_status(clear=True) == word   # the Python helper returns the word instead of raising
    assert _capi.device_status_result(clear=True) == (0, 0)
    # the next kernel runs normally
    a, b = oi.matmul_inputs(128, 128, 64, 31)
    out = torch.empty(128, 128, dtype=torch.float16, device="cuda")
    _capi.matmul(dev(a), dev(b), out)
    assert_close(host(out), ok.matmul(a, b))
    assert_device_healthy()
    with pytest.raises(_capi.KernelLaunchError):
        _capi.selftest_wait_timeout(limit_ns=0)


def test_launches_that_leave_the_tensor_core_path_say_so():
    from ninetoothed_b200 import _capi

    _capi.plain_launches(reset=True)
    a, b = oi.matmul_inputs(64, 64, 100, 32)  # K = 100: rows of 200 bytes, not addressable by TMA
    out = torch.empty(64, 64, dtype=torch.float16, device="cuda")
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        _capi.matmul(dev(a), dev(b), out)
    assert _capi.plain_launches() == 1
    assert any(issubclass(w.category, _capi.SlowPathWarning) and "plain CUDA-core kernel" in str(w.message) for w in caught)
    assert_close(host(out), ok.matmul(a, b))
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        a, b = oi.matmul_inputs(128, 128, 128, 33)
        out = torch.empty(128, 128, dtype=torch.float16, device="cuda")
        _capi.matmul(dev(a), dev(b), out)  # the fast path stays silent
    assert not caught and _capi.plain_launches() == 1
    assert_device_healthy()


def test_reserved_split_scratch_is_used_without_allocating_on_the_launch_path():
    from ninetoothed_b200 import _capi

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        _capi.reserve_split_scratch()
        _capi.reserve_split_scratch()  # idempotent
        a, b = oi.matmul_inputs(128, 256, 4096, 34)  # two tiles, long reduction: split along K
        out = torch.empty(128, 256, dtype=torch.float16, device="cuda")
        ad, bd = dev(a), dev(b)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _capi.matmul(ad, bd, out)
        torch.cuda.synchronize()
        assert free_before - torch.cuda.mem_get_info()[0] < (1 << 20)
    assert_close(host(out), ok.matmul(a, b, np.float16, 128, 256, 64))
    assert_device_healthy()
