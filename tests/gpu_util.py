"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

TORCH_DTYPE = {np.dtype(np.float16): torch.float16, np.dtype(np.float32): torch.float32}


def dev(array):
    """numpy array -> CUDA tensor (bit-exact copy)."""
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def host(tensor):
    return tensor.detach().cpu().numpy()


def assert_close(actual, expected, rtol=1e-2, atol=1e-2):
    """The parity bar for fp16/bf16 results: |a - e| <= atol + rtol * |e|."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape, (a.shape, e.shape)
    err = np.abs(a - e)
    bound = atol + rtol * np.abs(e)
    bad = err > bound
    if bad.any() or not np.isfinite(a).all():
        idx = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(
            f"{int(bad.sum())} of {a.size} elements out of tolerance; worst at {idx}: got {a[idx]!r}, "
            f"expected {e[idx]!r}; finite={bool(np.isfinite(a).all())}"
        )


def assert_device_healthy():
    from ninetoothed_b200 import _capi

    status = _capi.device_status(clear=True)
    assert status == 0, f"a bounded device-side wait gave up: status 0x{status:08x}"
