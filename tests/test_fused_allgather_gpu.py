"""addmm with the all-gather fused into the epilogue, on two GPUs of one node.

Each rank computes its column slab and the GEMM epilogue stores every tile into both ranks'
full-size buffers: with a plain store per rank over NVLink, and with one multimem.st to the
buffers' multicast mapping (the NVSwitch makes the copies) where the box has one.  Checked against the unfused path (local addmm +
NCCL all-gather) bit for bit, and against the oracle on rank 0.  Skipped on a single-GPU box.
"""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, through_switch, results):
    import torch.distributed as dist

    from ninetoothed_b200 import _capi, sharding
    from oracle import inputs as oi
    from oracle import kernels as ok

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        m, n, k = 2304, 4608, 512  # enough tiles for the CTA-pair kernel on each rank's 2304-column slab
        c, a, b = oi.addmm_inputs(m, n, k, 77)
        cols = sharding.even_slab(n, rank, world)
        c_slab = torch.from_numpy(np.ascontiguousarray(c[:, cols])).to(device)
        b_slab = torch.from_numpy(np.ascontiguousarray(b[:, cols])).to(device)
        a_dev = torch.from_numpy(a).to(device)
        probe = sharding.GatheredColumns(m, n, torch.float16, device)
        if through_switch and not probe.multicast_slab_ptr:
            results[rank] = "no multicast mapping"
            return
        gathered = sharding.GatheredColumns(m, n, torch.float16, device, through_switch=through_switch)
        assert gathered.through_switch == through_switch
        ok_all = True
        for _ in range(2):  # twice: the second call overwrites a buffer that is already full
            gathered.full.zero_()
            dist.barrier()
            gathered.addmm(c_slab, a_dev, b_slab, 0.5, 2.0)
            full = gathered.wait()
            local = torch.empty(m, cols.stop - cols.start, dtype=torch.float16, device=device)
            _capi.addmm(c_slab, a_dev, b_slab, 0.5, 2.0, local)
            reference = sharding.gather_columns(local)
            ok_all = ok_all and bool(torch.equal(full, reference))
        expected = ok.addmm(c, a, b, 0.5, 2.0, np.float16, 256, 256, 64)
        close = np.abs(full.cpu().numpy().astype(np.float32) - expected.astype(np.float32)) <= 1e-2 + 1e-2 * np.abs(
            expected.astype(np.float32))
        results[rank] = (ok_all, bool(close.all()), _capi.device_status())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("through_switch", [False, True], ids=["peer_stores", "through_switch"])
def test_two_ranks_fill_each_others_buffers(through_switch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), through_switch, results), nprocs=world, join=True)
    if through_switch and set(results.values()) == {"no multicast mapping"}:
        pytest.skip("the symmetric allocation has no multicast mapping on this box")
    assert dict(results) == {0: (True, True, 0), 1: (True, True, 0)}
