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


def test_overlapping_steps_keep_their_inputs_and_outputs_apart():
    """With ``overlap_steps`` a step's copies in start while the previous step's last kernel and copies out are still
    running: four steps on different inputs, each into its own host buffer, nothing synchronised in between."""
    from ninetoothed_b200.host_pipeline import HostAddmm

    m, n, k = 1152, 512, 320
    pipeline = HostAddmm(kd.make_addmm(), m, n, k, torch.float16, "cuda", row_block=256, overlap_steps=True)
    steps = []
    for seed, (beta, alpha) in ((21, (1.0, 1.0)), (22, (0.5, -2.0)), (23, (0.0, 1.0)), (24, (2.0, 0.25))):
        c, a, b = oi.addmm_inputs(m, n, k, seed)
        host = [torch.from_numpy(x).pin_memory() for x in (c, a, b)]
        steps.append((c, a, b, beta, alpha, host, torch.empty(m, n, dtype=torch.float16).pin_memory()))
    for c, a, b, beta, alpha, host, out_host in steps:
        pipeline(host[0], host[1], host[2], beta, alpha, out_host)
    pipeline.wait()
    torch.cuda.current_stream().synchronize()
    for c, a, b, beta, alpha, host, out_host in steps:
        assert_close(out_host.numpy(), ok.addmm(c, a, b, beta, alpha))
    assert_device_healthy()


def test_shape_mismatch_is_rejected():
    from ninetoothed_b200.host_pipeline import HostAddmm

    pipeline = HostAddmm(kd.make_addmm(), 128, 128, 64, torch.float16, "cuda")
    good = torch.empty(128, 128, dtype=torch.float16)
    with pytest.raises(ValueError):
        pipeline(good, torch.empty(128, 32, dtype=torch.float16), torch.empty(64, 128, dtype=torch.float16), 1.0, 1.0,
                 good)


def _free_port():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _sharded_worker(rank, world, port, results):
    import os

    import numpy as np
    import torch.distributed as dist

    from ninetoothed_b200 import sharding
    from ninetoothed_b200.host_pipeline import ShardedHostAddmm

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        m, n, k = 512, 768, 256
        cols = sharding.even_slab(n, rank, world)
        pipeline = ShardedHostAddmm(kd.make_addmm(), m, cols.stop - cols.start, k, torch.float16, device, row_block=128)
        good = True
        for seed in (61, 62):  # twice: the second step reuses the staging buffers
            c, a, b = oi.addmm_inputs(m, n, k, seed)
            host_c = torch.from_numpy(np.ascontiguousarray(c[:, cols])).pin_memory()
            host_b = torch.from_numpy(np.ascontiguousarray(b[:, cols])).pin_memory()
            host_a_rows = torch.from_numpy(np.ascontiguousarray(a[pipeline.rows])).pin_memory()  # 1/world of mat1
            out_host = torch.empty(m, cols.stop - cols.start, dtype=torch.float16).pin_memory()
            pipeline(host_c, host_a_rows, host_b, 0.5, 2.0, out_host)
            torch.cuda.synchronize()
            expected = ok.addmm(c[:, cols], a, b[:, cols], 0.5, 2.0).astype(np.float32)
            good = good and bool((np.abs(out_host.numpy().astype(np.float32) - expected)
                                  <= 1e-2 + 1e-2 * np.abs(expected)).all())
        # and three steps that overlap (nothing synchronised in between, each into its own host buffer)
        overlapped = ShardedHostAddmm(kd.make_addmm(), m, cols.stop - cols.start, k, torch.float16, device,
                                      row_block=128, overlap_steps=True)
        steps = []
        for seed in (63, 64, 65):
            c, a, b = oi.addmm_inputs(m, n, k, seed)
            hosts = [torch.from_numpy(np.ascontiguousarray(x)).pin_memory()
                     for x in (c[:, cols], a[overlapped.rows], b[:, cols])]
            steps.append((c, a, b, hosts, torch.empty(m, cols.stop - cols.start, dtype=torch.float16).pin_memory()))
        for c, a, b, hosts, out_host in steps:
            overlapped(hosts[0], hosts[1], hosts[2], 0.5, 2.0, out_host)
        overlapped.wait()
        torch.cuda.synchronize()
        for c, a, b, hosts, out_host in steps:
            expected = ok.addmm(c[:, cols], a, b[:, cols], 0.5, 2.0).astype(np.float32)
            good = good and bool((np.abs(out_host.numpy().astype(np.float32) - expected)
                                  <= 1e-2 + 1e-2 * np.abs(expected)).all())
        results[rank] = (good, pipeline.h2d_bytes() == (m // world * k + k * (n // world) + m * (n // world)) * 2)
    finally:
        dist.destroy_process_group()


def test_sharded_step_brings_in_one_share_of_mat1_per_rank():
    """Two ranks: each copies in half of mat1's rows and gathers the other half from its peer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_sharded_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}
