"""Multi-rank host logic on CPU: world size 2, gloo backend.

The kernels shard by independent output units; these tests run the partition and
the all-gather helpers of ninetoothed_b200.sharding in two processes, with the numpy
oracle standing in for the CUDA kernel, and check the reassembled output against the
unsharded result.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ninetoothed_b200 import sharding
from oracle import inputs as oi
from oracle import kernels as ok


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # addmm: N-columns; A replicated, B and C column slabs, output slabs all-gathered
        m, n, k = 96, 128, 64
        c, a, b = oi.addmm_inputs(m, n, k, 5)
        cols = sharding.even_slab(n, rank, world)
        local = ok.addmm(c[:, cols], a, b[:, cols], 0.5, 2.0, np.float16, 32, 32, 32)
        full = sharding.gather_columns(torch.from_numpy(local))
        expected = ok.addmm(c, a, b, 0.5, 2.0, np.float16, 32, 32, 32)
        ok_addmm = np.array_equal(full.numpy(), expected)

        # conv2d: batch slabs, contiguous, gathered along dim 0
        x, w = oi.conv2d_inputs((4, 8, 6, 6), (16, 8, 3, 3), 6)
        images = sharding.even_slab(4, rank, world)
        local = ok.conv2d(x[images], w, (1, 1), block_m=32, block_n=32, block_k=32)
        full = sharding.gather_leading(torch.from_numpy(local))
        ok_conv = np.array_equal(full.numpy(), ok.conv2d(x, w, (1, 1), block_m=32, block_n=32, block_k=32))

        # attention: (batch, head) pairs
        q, kk, v = (torch.from_numpy(t) for t in oi.attention_inputs((2, 2, 16, 8), 7))
        ql, kl, vl = (sharding.attention_slab(t, rank, world) for t in (q, kk, v))
        local = ok.attention(ql.numpy(), kl.numpy(), vl.numpy(), True, 8, 8)
        full = sharding.gather_leading(torch.from_numpy(local)).reshape(2, 2, 16, 8)
        ok_attn = np.array_equal(full.numpy(), ok.attention(q.numpy(), kk.numpy(), v.numpy(), True, 8, 8))

        # a replicated operand that starts in host memory: every rank brings in its rows, the rest is gathered
        whole = torch.from_numpy(a)
        mine = whole[sharding.even_slab(m, rank, world)]
        gathered = sharding.gather_rows_into(torch.empty_like(whole), mine)
        ok_rows_gathered = bool(torch.equal(gathered, whole))
        try:
            sharding.gather_rows_into(torch.empty(m + 1, k, dtype=whole.dtype), mine)
            ok_rows_gathered = False
        except ValueError:
            pass

        # softmax: rows stay sharded; the union of the slabs covers every row once
        rows = sharding.slab(10, rank, world)
        counts = torch.zeros(10, dtype=torch.int64)
        counts[rows] += 1
        dist.all_reduce(counts)
        ok_rows = bool((counts == 1).all())
        results[rank] = (ok_addmm, ok_conv, ok_attn, ok_rows and ok_rows_gathered)
    finally:
        dist.destroy_process_group()


def test_world_size_two_reassembles_every_kernel():
    world = 2
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: (True, True, True, True), 1: (True, True, True, True)}


def test_slab_arithmetic():
    assert [sharding.slab(10, r, 4) for r in range(4)] == [slice(0, 3), slice(3, 6), slice(6, 8), slice(8, 10)]
    assert sharding.even_slab(8192, 3, 8) == slice(3072, 4096)
    with pytest.raises(ValueError):
        sharding.even_slab(10, 0, 4)
    covered = sorted(i for r in range(3) for i in range(*sharding.slab(7, r, 3).indices(7)))
    assert covered == list(range(7))
