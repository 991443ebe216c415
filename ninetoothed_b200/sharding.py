"""Partitioning of the four kernels across the GPUs of one node.

The kernels have independent output units, so each rank computes a slab and at
most one exchange follows: an all-gather of the output slabs, only when the full
output is wanted on every rank.

    matmul / addmm   N-columns: rank r owns out[:, r*N/g : (r+1)*N/g]
    conv2d           batch:     rank r owns y[r*B/g : (r+1)*B/g]
    attention        batch x head pairs, contiguous in [B, H, S, D]
    softmax          rows (never gathered: the result is consumed where it is)

One process per GPU; the collective is ``torch.distributed.all_gather_into_tensor``
(NCCL over NVLink on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def slab(total: int, rank: int, world_size: int) -> slice:
    """Contiguous, near-even split of ``total`` units; the first ``total % world_size`` ranks take one more."""
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def even_slab(total: int, rank: int, world_size: int) -> slice:
    if total % world_size:
        raise ValueError(f"{total} units do not split evenly over {world_size} ranks")
    width = total // world_size
    return slice(rank * width, (rank + 1) * width)


def _all_gather_stacked(stacked: torch.Tensor, local: torch.Tensor, group=None) -> None:
    """stacked[r] <- rank r's ``local``.  NCCL gathers straight into the buffer; backends
    without that primitive (gloo, in the CPU tests) gather into its slices."""
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(stacked, local, group=group)
    else:
        dist.all_gather([stacked[r] for r in range(stacked.shape[0])], local, group=group)


def gather_leading(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather slabs that split dimension 0 (conv2d batch, softmax rows, attention
    batch*head after flattening): the gathered buffer IS the full tensor."""
    world_size = dist.get_world_size(group)
    local = local.contiguous()
    stacked = torch.empty((world_size,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    _all_gather_stacked(stacked, local, group)
    return stacked.reshape((world_size * local.shape[0],) + tuple(local.shape[1:]))


def gather_columns(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather [M, N/g] column slabs into the row-major [M, N] matrix.

    The collective delivers [g, M, N/g]; one strided copy re-lays it out."""
    world_size = dist.get_world_size(group)
    local = local.contiguous()
    m, width = local.shape
    stacked = torch.empty((world_size, m, width), dtype=local.dtype, device=local.device)
    _all_gather_stacked(stacked, local, group)
    return stacked.permute(1, 0, 2).reshape(m, world_size * width)


def attention_slab(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Rank's share of the B*H (batch, head) pairs of a contiguous [B, H, S, D] tensor, as [pairs, 1, S, D]."""
    b, h, s, d = t.shape
    pairs = t.reshape(b * h, 1, s, d)
    return pairs[even_slab(b * h, rank, world_size)]
