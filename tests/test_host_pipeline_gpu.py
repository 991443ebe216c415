"""addmm from host memory with the copies pipelined (ninetoothed_b200/host_pipeline.py).

Two steps in a row on different inputs through one pipeline (the second step reuses
the staging buffers, so the cross-step ordering is exercised), a ragged last row
block, against the oracle.  Tolerance: the fp16 bar, rtol 1e-2 / atol 1e-2.
"""

import pytest
import torch

from examples import definitions as kd
from oracle import inputs as oi
from oracle import kernels as ok

from gpu_util import assert_close, assert_device_healthy

pytestmark = pytest.mark.gpu


def test_two_steps_through_one_pipeline():
    from ninetoothed_b200.host_pipeline import HostAddmm

    m, n, k = 640, 256, 192
    pipeline = HostAddmm(kd.make_addmm(), m, n, k, torch.float16, "cuda", row_block=256)
    assert [b.stop - b.start for b in pipeline.blocks] == [256, 256, 128]
    out_host = torch.empty(m, n, dtype=torch.float16).pin_memory()
    for seed, (beta, alpha) in ((11, (1.0, 1.0)), (12, (0.5, -2.0))):
        c, a, b = oi.addmm_inputs(m, n, k, seed)
        host = [torch.from_numpy(x).pin_memory() for x in (c, a, b)]
        pipeline(host[0], host[1], host[2], beta, alpha, out_host)
        torch.cuda.synchronize()
        assert_close(out_host.numpy(), ok.addmm(c, a, b, beta, alpha))
    assert_device_healthy()


def test_shape_mismatch_is_rejected():
    from ninetoothed_b200.host_pipeline import HostAddmm

    pipeline = HostAddmm(kd.make_addmm(), 128, 128, 64, torch.float16, "cuda")
    good = torch.empty(128, 128, dtype=torch.float16)
    with pytest.raises(ValueError):
        pipeline(good, torch.empty(128, 32, dtype=torch.float16), torch.empty(64, 128, dtype=torch.float16), 1.0, 1.0,
                 good)
