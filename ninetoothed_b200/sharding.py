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


def gather_rows_into(full: torch.Tensor, local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather equal row slabs of a replicated operand into the preallocated ``full`` matrix:
    rank r contributes rows [r*M/g, (r+1)*M/g).  Used when every rank needs the whole of a matrix that
    starts out in host memory: each rank brings in 1/g of it and the rest arrives over NVLink."""
    world_size = dist.get_world_size(group)
    rows = local.shape[0]
    if full.shape[0] != rows * world_size or tuple(full.shape[1:]) != tuple(local.shape[1:]):
        raise ValueError(f"cannot gather {world_size} slabs of shape {tuple(local.shape)} into {tuple(full.shape)}")
    _all_gather_stacked(full.view((world_size, rows) + tuple(full.shape[1:])), local.contiguous(), group)
    return full


def gather_columns(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather [M, N/g] column slabs into the row-major [M, N] matrix.

    The collective delivers [g, M, N/g]; one strided copy re-lays it out."""
    world_size = dist.get_world_size(group)
    local = local.contiguous()
    m, width = local.shape
    stacked = torch.empty((world_size, m, width), dtype=local.dtype, device=local.device)
    _all_gather_stacked(stacked, local, group)
    return stacked.permute(1, 0, 2).reshape(m, world_size * width)


def multicast_slab_layout_ok(slab: torch.Tensor) -> bool:
    """Whether ``launch_addmm_allgather_multicast`` takes this [M, N_local] slab (as output or as addmm input):
    whole 64-column steps, unit-stride rows, 16-byte aligned rows."""
    elements = 16 // slab.element_size()
    return (
        slab.dim() == 2
        and slab.shape[1] % 64 == 0
        and slab.stride(1) == 1
        and slab.stride(0) % elements == 0
        and slab.data_ptr() % 16 == 0
    )


class GatheredColumns:
    """The full [M, N] output of a column-split addmm, on every rank, filled by the fused kernel.

    Each rank allocates its [M, N] buffer in symmetric memory (one allocation per rank, mapped
    into every other rank's address space over NVLink) and ``addmm`` runs
    ``launch_addmm_allgather``: the GEMM epilogue stores each tile of the rank's column slab into
    all the buffers, so no separate collective moves the output.  ``wait`` is the barrier after
    which every rank's ``full`` holds the whole matrix.

    ``through_switch``: where the symmetric allocation is bound to an NVLink multicast object (the handle's
    ``multicast_ptr`` is non-zero) and the slab's layout allows it, each tile is stored once to the multicast
    address (``launch_addmm_allgather_multicast``) and the NVSwitch writes it into every rank's buffer; otherwise
    the kernel stores to each peer's buffer itself.  ``None`` picks the multicast path when it is available.
    """

    def __init__(self, m: int, n: int, dtype, device, group=None, through_switch=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.full = symm_mem.empty((m, n), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.full, self.group)
        self.peer_ptrs = [int(ptr) for ptr in self.handle.buffer_ptrs]
        self.columns = even_slab(n, self.rank, self.world)
        self.slab = self.full[:, self.columns]
        multicast_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        can_multicast = multicast_base != 0 and self.world > 1 and multicast_slab_layout_ok(self.slab)
        if through_switch and not can_multicast:
            raise RuntimeError(
                "the symmetric allocation has no multicast mapping (or the slab is not whole 64-column steps of "
                "16-byte aligned rows): the switch cannot make the copies here"
            )
        self.through_switch = can_multicast if through_switch is None else bool(through_switch)
        # the slab sits at the same byte offset in the multicast mapping as in this rank's own buffer
        self.multicast_slab_ptr = multicast_base + (self.slab.data_ptr() - self.full.data_ptr()) if can_multicast else 0

    def addmm(self, input_slab, mat1, mat2_slab, beta=1.0, alpha=1.0):
        from ninetoothed_b200 import _capi

        if self.through_switch and multicast_slab_layout_ok(input_slab):
            _capi.addmm_allgather_multicast(input_slab, mat1, mat2_slab, beta, alpha, self.slab, self.multicast_slab_ptr)
        else:
            _capi.addmm_allgather(input_slab, mat1, mat2_slab, beta, alpha, self.slab, self.peer_ptrs, self.rank)

    def wait(self):
        """All ranks' tiles have landed in this rank's buffer (and this rank's in theirs)."""
        self.handle.barrier()
        return self.full


def attention_slab(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Rank's share of the B*H (batch, head) pairs of a contiguous [B, H, S, D] tensor, as [pairs, 1, S, D]."""
    b, h, s, d = t.shape
    pairs = t.reshape(b * h, 1, s, d)
    return pairs[even_slab(b * h, rank, world_size)]
