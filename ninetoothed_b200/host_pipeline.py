"""addmm on operands that live in host memory, with the PCIe copies overlapped.

A caller whose matrices are in (pinned) host memory pays far more for the copies
than for the kernel: an 8192^3 fp16 addmm moves 403 MB in and 134 MB out at
~55 GB/s per direction against under a millisecond of tensor-core time.  The two
PCIe directions are independent, and the kernel only needs the rows of ``mat1``
and ``input`` it is working on, so ``HostAddmm`` cuts the problem into row blocks
and runs three streams:

    copy-in    mat2 whole, then for each row block: mat1[rows], input[rows]
    compute    the addmm kernel handle on (input[rows], mat1[rows], mat2) -> out[rows]
    copy-out   out[rows] back to the host buffer

so that the step costs about the host-to-device time alone.  Every block goes
through the same kernel handle a user gets from ``make`` (the reference-facing
call); nothing here computes.
"""

from __future__ import annotations

import torch


class HostAddmm:
    """``out_host = beta * input_host + alpha * mat1_host @ mat2_host`` for fixed shapes.

    Device staging buffers, streams and events are created once; ``__call__`` enqueues
    one step and returns without synchronising: when the caller's current stream has
    finished, ``out_host`` holds the result.  Host tensors should be pinned, otherwise
    the copies are synchronous and nothing overlaps.

    ``overlap_steps=True`` lets consecutive steps overlap as well: a step's copies in then wait
    only for the previous step's kernels (which read the staging buffers), not for its last
    copies out, so the tail of one step (last block's kernel and copy out) runs under the next
    step's copies in.  The caller's stream is then NOT made to wait for the copies out: call
    ``wait()`` (or synchronise the device) before reading ``out_host``, and have the host
    inputs complete before each call (they are read on the pipeline's own stream, which is
    ordered after the pipeline's previous step only)."""

    def __init__(self, kernel, m: int, n: int, k: int, dtype, device, row_block: int = 1024,
                 overlap_steps: bool = False):
        self.overlap_steps = overlap_steps
        self.kernels_done = None  # recorded after a step's last kernel (overlap_steps only)
        self.m, self.n, self.k = m, n, k
        self.device = torch.device(device)
        self.kernel = kernel  # the addmm handle from make(): kernel(input, mat1, mat2, beta, alpha, output)
        self.blocks = [slice(r, min(r + row_block, m)) for r in range(0, m, row_block)]
        self.input = torch.empty(m, n, dtype=dtype, device=self.device)
        self.mat1 = torch.empty(m, k, dtype=dtype, device=self.device)
        self.mat2 = torch.empty(k, n, dtype=dtype, device=self.device)
        self.out = torch.empty(m, n, dtype=dtype, device=self.device)
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self.arrived = [torch.cuda.Event() for _ in self.blocks]
        self.computed = [torch.cuda.Event() for _ in self.blocks]
        self.copied_out = [torch.cuda.Event() for _ in self.blocks]

    def wait(self):
        """The caller's current stream waits for every copy out enqueued so far."""
        torch.cuda.current_stream(self.device).wait_stream(self.copy_out)

    def __call__(self, input_host, mat1_host, mat2_host, beta, alpha, out_host):
        for name, t, shape in (("input", input_host, (self.m, self.n)), ("mat1", mat1_host, (self.m, self.k)),
                               ("mat2", mat2_host, (self.k, self.n)), ("output", out_host, (self.m, self.n))):
            if tuple(t.shape) != shape:
                raise ValueError(f"{name} has shape {tuple(t.shape)}, this pipeline was built for {shape}")
        main = torch.cuda.current_stream(self.device)
        # The previous step's kernels must be done with the staging buffers before they are
        # overwritten, and its copies out of `out` before `out` is written again.
        overlapping = self.overlap_steps and self.kernels_done is not None
        if overlapping:
            self.copy_in.wait_event(self.kernels_done)
        else:
            self.copy_in.wait_stream(main)
            main.wait_stream(self.copy_out)
        with torch.cuda.stream(self.copy_in):
            self.mat2.copy_(mat2_host, non_blocking=True)
        for rows, arrived, computed, copied_out in zip(self.blocks, self.arrived, self.computed, self.copied_out):
            with torch.cuda.stream(self.copy_in):
                self.mat1[rows].copy_(mat1_host[rows], non_blocking=True)
                self.input[rows].copy_(input_host[rows], non_blocking=True)
                arrived.record(self.copy_in)
            main.wait_event(arrived)
            if overlapping:
                main.wait_event(copied_out)  # the previous step's copy of these rows of `out` has left the device
            self.kernel(self.input[rows], self.mat1[rows], self.mat2, beta, alpha, self.out[rows])
            computed.record(main)
            self.copy_out.wait_event(computed)
            with torch.cuda.stream(self.copy_out):
                out_host[rows].copy_(self.out[rows], non_blocking=True)
                copied_out.record(self.copy_out)
        if self.overlap_steps:
            self.kernels_done = torch.cuda.Event()
            self.kernels_done.record(main)
        else:
            main.wait_stream(self.copy_out)
        return out_host


class ShardedHostAddmm:
    """The same step on g ranks that split the N-columns: rank r owns ``out[:, cols_r]``.

    ``mat1`` is needed whole by every rank.  Copying it to every GPU from the host would move g copies
    over the host's memory system and PCIe; here every rank copies in only rows
    [r*M/g, (r+1)*M/g) of it and the ranks all-gather the rest over NVLink
    (``sharding.gather_rows_into``), while their ``mat2`` and ``input`` column slabs are still crossing
    PCIe.  The row blocks of the output then go back to the host as they are computed.
    Per step and rank the host sends M*K/g + K*N/g + M*N/g elements and receives M*N/g.
    ``overlap_steps`` as in ``HostAddmm``: consecutive steps overlap, ``wait()`` joins the copies out.
    """

    def __init__(self, kernel, m: int, n_local: int, k: int, dtype, device, group=None, row_block: int = 1024,
                 overlap_steps: bool = False):
        import torch.distributed as dist

        self.overlap_steps = overlap_steps
        self.kernels_done = None

        from ninetoothed_b200 import sharding

        self.kernel = kernel
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.m, self.n_local, self.k = m, n_local, k
        self.rows = sharding.even_slab(m, self.rank, self.world)  # the rows of mat1 this rank brings in
        self.device = torch.device(device)
        self.blocks = [slice(r, min(r + row_block, m)) for r in range(0, m, row_block)]
        self.input = torch.empty(m, n_local, dtype=dtype, device=self.device)
        self.mat1 = torch.empty(m, k, dtype=dtype, device=self.device)
        self.mat1_rows = torch.empty(self.rows.stop - self.rows.start, k, dtype=dtype, device=self.device)
        self.mat2 = torch.empty(k, n_local, dtype=dtype, device=self.device)
        self.out = torch.empty(m, n_local, dtype=dtype, device=self.device)
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self.rows_arrived = torch.cuda.Event()
        self.arrived = [torch.cuda.Event() for _ in self.blocks]
        self.computed = [torch.cuda.Event() for _ in self.blocks]
        self.copied_out = [torch.cuda.Event() for _ in self.blocks]

    def wait(self):
        """The caller's current stream waits for every copy out enqueued so far."""
        torch.cuda.current_stream(self.device).wait_stream(self.copy_out)

    def h2d_bytes(self):
        return (self.mat1_rows.numel() + self.mat2.numel() + self.input.numel()) * self.mat1.element_size()

    def d2h_bytes(self):
        return self.out.numel() * self.out.element_size()

    def __call__(self, input_host, mat1_rows_host, mat2_host, beta, alpha, out_host):
        """``mat1_rows_host`` holds this rank's rows of mat1 only; the other arguments are its column slabs."""
        from ninetoothed_b200 import sharding

        main = torch.cuda.current_stream(self.device)
        overlapping = self.overlap_steps and self.kernels_done is not None
        if overlapping:
            self.copy_in.wait_event(self.kernels_done)  # the staging buffers are free once the last kernel has run
        else:
            self.copy_in.wait_stream(main)
            main.wait_stream(self.copy_out)
        with torch.cuda.stream(self.copy_in):
            self.mat1_rows.copy_(mat1_rows_host, non_blocking=True)
            self.rows_arrived.record(self.copy_in)
            self.mat2.copy_(mat2_host, non_blocking=True)
        main.wait_event(self.rows_arrived)
        sharding.gather_rows_into(self.mat1, self.mat1_rows, self.group)  # over NVLink, under the copies above
        for rows, arrived, computed, copied_out in zip(self.blocks, self.arrived, self.computed, self.copied_out):
            with torch.cuda.stream(self.copy_in):
                self.input[rows].copy_(input_host[rows], non_blocking=True)
                arrived.record(self.copy_in)
            main.wait_event(arrived)
            if overlapping:
                main.wait_event(copied_out)  # the previous step's copy of these rows of `out` has left the device
            self.kernel(self.input[rows], self.mat1[rows], self.mat2, beta, alpha, self.out[rows])
            computed.record(main)
            self.copy_out.wait_event(computed)
            with torch.cuda.stream(self.copy_out):
                out_host[rows].copy_(self.out[rows], non_blocking=True)
                copied_out.record(self.copy_out)
        if self.overlap_steps:
            self.kernels_done = torch.cuda.Event()
            self.kernels_done.record(main)
        else:
            main.wait_stream(self.copy_out)
        return out_host
