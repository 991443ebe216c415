#!/usr/bin/env python
"""Throughput of the B200 kernels behind the NineToothed operator API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload: addmm fp16, out = beta*C + alpha*(A.B) with M=N=K=8192,
alpha=beta=1, seeded N(0,1) inputs.  One step = one pass of that kernel.  With N
GPUs the N columns are split over the ranks (A replicated, B and C column slabs) with
no collective on the data path, so the total work is fixed ("strong" scaling); the
same step with the column slabs all-gathered onto every rank is timed beside it, both
fused into the GEMM epilogue (peer stores over NVLink) and through NCCL.  Rank 0 prints ONE JSON line:

  value      whole-job TFLOP/s with inputs resident in HBM, CUDA-event timed,
             max over ranks
  e2e        the same step through the public API (the callable `make` returns)
             with HOST buffers: pinned H2D of the inputs and D2H of the result
             inside the timed region
  roofline   the GEMM kernel alone against the measured tensor peak
  cpu_baseline  the numpy port of the reference's algorithm on the host cores
  ops        the other kernels of the metric (softmax GB/s, attention and conv2d
             TFLOP/s) at their benchmark shapes, sharded over the same ranks

`--impl reference` times the CPU port of the reference's algorithm (the oracle) on
the host cores instead; only rank 0 works.
Inputs (4 x 128 MiB) exceed the 126 MB L2, so no flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SIZE = 8192
FLOPS = 2.0 * SIZE**3
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel,
# from the ncu capture summarised under profiles/.
NCU_TRAFFIC_BYTES = {"gemm_8192": 1264872000 + 126561536}  # profiles/gemm_addmm_8192_fp16.md
_RESULT_STREAM = sys.stdout  # where the one result line goes (see main)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the `with` body runs: through NVML
    every 2 ms when the bindings are importable (a timed region of 20 launches lasts ~15 ms), else through
    `nvidia-smi -lms 100`.  Read-only: nothing about the GPU is set."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NVML_REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"),
                    (0x4, "sw_power_cap"))

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None
        self.samples, self.sm_max, self.reasons, self.source = [], None, set(), None
        self._stop = threading.Event()
        self.thread = None

    def _nvml_handle(self):
        import pynvml
        import torch

        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll_nvml(self, pynvml, handle):
        while not self._stop.is_set():
            try:
                self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                mask = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                for bit, name in self.NVML_REASONS:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        try:
            pynvml, handle = self._nvml_handle()
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.source = "nvml, every 2 ms"
            self.thread = threading.Thread(target=self._poll_nvml, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.source = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi, every 100 ms"
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        sm, sm_max, reasons = list(self.samples), [self.sm_max] if self.sm_max else [], set(self.reasons)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(sm_max) if sm_max else None,
                "sm_min_mhz": min(sm), "reasons": sorted(reasons), "samples": len(sm), "source": self.source}


# ----------------------------------------------------------------------------
# CPU arm: the numpy port of the reference's algorithm
# ----------------------------------------------------------------------------
def host_threads():
    try:
        from threadpoolctl import threadpool_info

        counts = [pool.get("num_threads", 1) for pool in threadpool_info() if pool.get("user_api") == "blas"]
        return max(counts) if counts else os.cpu_count()
    except Exception:
        return os.cpu_count()


def cpu_addmm_rate(n, repeats=1):
    """TFLOP/s of oracle.kernels.addmm on an n^3 sample (fp16 in, fp32 accumulate)."""
    import numpy as np

    from oracle import inputs as oi
    from oracle import kernels as ok

    c, a, b = oi.addmm_inputs(n, n, n, 1)
    block = min(n, 1024)
    best = math.inf
    for _ in range(repeats):
        t0 = time.perf_counter()
        ok.addmm(c, a, b, 1.0, 1.0, np.float16, block, block, block)
        best = min(best, time.perf_counter() - t0)
    return 2.0 * n**3 / best / 1e12, best


def cpu_baseline(target_seconds=12.0):
    import numpy  # noqa: F401  (BLAS pool must exist before counting its threads)

    rate, _ = cpu_addmm_rate(1024)
    n = 2048
    while n < SIZE and 2.0 * (2 * n) ** 3 / (rate * 1e12) < target_seconds:
        n *= 2
    rate, seconds = cpu_addmm_rate(n)
    return {"value": rate, "unit": "TFLOP/s", "cores": host_threads(), "kind": "port",
            "sample": f"oracle.kernels.addmm (numpy, fp32 accumulate) on one {n}^3 fp16 problem, {seconds:.2f} s; "
                      "rate counted with that problem's own 2*n^3 FLOPs"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = 2048
    rate, _ = cpu_addmm_rate(1024)
    while n < 4096 and (args.steps + args.warmup) * 2.0 * (2 * n) ** 3 / (rate * 1e12) < 90.0:
        n *= 2
    for _ in range(args.warmup):
        cpu_addmm_rate(n)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_addmm_rate(n)
    elapsed = time.perf_counter() - t0
    value = args.steps * 2.0 * n**3 / elapsed / 1e12
    sample = f"oracle.kernels.addmm (numpy port of the reference's tiled loop) on a {n}^3 fp16 sample per step"
    line = {
        "impl": "reference", "metric": "fp16 addmm TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"addmm fp16 M=N=K={SIZE}, alpha=beta=1 (bounded sample: {n}^3 per step)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": host_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=_RESULT_STREAM, flush=True)


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------
def run_b200(args):
    import torch
    import torch.distributed as dist

    from examples import definitions as kd
    from ninetoothed_b200 import _capi, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _capi.library()  # fail here, loudly, if the CUDA library is missing

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- inputs: rank r owns N-columns [r*N/g, (r+1)*N/g) --------------------
    cols = sharding.even_slab(SIZE, rank, world)
    width = cols.stop - cols.start
    gen = torch.Generator(device=device).manual_seed(1)
    c_full = torch.randn(SIZE, SIZE, generator=gen, device=device, dtype=torch.float32).half()
    a = torch.randn(SIZE, SIZE, generator=gen, device=device, dtype=torch.float32).half()
    b_full = torch.randn(SIZE, SIZE, generator=gen, device=device, dtype=torch.float32).half()
    c_in = c_full[:, cols].contiguous()
    b = b_full[:, cols].contiguous()
    del c_full, b_full
    out = torch.empty(SIZE, width, dtype=torch.float16, device=device)
    addmm_kernel = kd.make_addmm()
    # N > 1: the all-gather of the column slabs is fused into the GEMM epilogue (peer stores over
    # NVLink into every rank's full-size buffer); the NCCL all-gather is measured beside it.
    gathered = sharding.GatheredColumns(SIZE, SIZE, torch.float16, device) if world > 1 else None
    fused_matches_nccl = None
    if world > 1:
        gathered.addmm(c_in, a, b, 1.0, 1.0)
        full_fused = gathered.wait().clone()
        _capi.addmm(c_in, a, b, 1.0, 1.0, out)
        fused_matches_nccl = bool(torch.equal(full_fused, sharding.gather_columns(out)))
        del full_fused

    def step():
        _capi.addmm(c_in, a, b, 1.0, 1.0, out)
        return out

    kernel_events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                     for _ in range(args.steps)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:  # samples every 100 ms over the warm-up and the timed steps
        for _ in range(max(args.warmup, 3)):
            step()
        barrier()
        start.record()
        for k0, k1 in kernel_events:
            k0.record()
            _capi.addmm(c_in, a, b, 1.0, 1.0, out)
            k1.record()
        end.record()
        barrier()
    total_ms = max_over_ranks(start.elapsed_time(end))
    kernel_ms = statistics.mean(k0.elapsed_time(k1) for k0, k1 in kernel_events)
    value = args.steps * FLOPS / (total_ms * 1e-3) / 1e12
    status = _capi.device_status()

    # ---- for N > 1: the same step with the column slabs reassembled on every rank, two ways -----
    fused_value = nccl_value = None
    if world > 1:
        barrier()
        start.record()
        for _ in range(args.steps):
            gathered.addmm(c_in, a, b, 1.0, 1.0)
            gathered.wait()
        end.record()
        barrier()
        fused_value = args.steps * FLOPS / (max_over_ranks(start.elapsed_time(end)) * 1e-3) / 1e12
        start.record()
        for _ in range(args.steps):
            _capi.addmm(c_in, a, b, 1.0, 1.0, out)
            sharding.gather_columns(out)
        end.record()
        barrier()
        nccl_value = args.steps * FLOPS / (max_over_ranks(start.elapsed_time(end)) * 1e-3) / 1e12

    # ---- the same kernel back to back for about a second: clocks under sustained load ----------
    sustained_launches = 3 if args.no_sustained else max(50, int(1.0 / (kernel_ms * 1e-3)))
    with ClockSampler(local_rank) as sustained_clocks:
        barrier()
        start.record()
        for _ in range(sustained_launches):
            _capi.addmm(c_in, a, b, 1.0, 1.0, out)
        end.record()
        barrier()
    sustained_ms = max_over_ranks(start.elapsed_time(end))
    sustained_value = sustained_launches * FLOPS / (sustained_ms * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers -------------------
    # The handle returned by make() is called on row blocks while the next block's operands and
    # the previous block's result cross PCIe on their own streams (ninetoothed_b200.host_pipeline);
    # the plain sequence copy-in, one call, copy-out is timed beside it.
    from ninetoothed_b200.host_pipeline import HostAddmm

    host_c, host_a, host_b = (t.cpu().pin_memory() for t in (c_in, a, b))
    host_out = torch.empty(SIZE, width, dtype=torch.float16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (host_c, host_a, host_b))
    d2h = host_out.numel() * host_out.element_size()
    pipeline = HostAddmm(addmm_kernel, SIZE, width, SIZE, torch.float16, device, row_block=1024)

    def e2e_step():
        pipeline(host_c, host_a, host_b, 1.0, 1.0, host_out)

    def e2e_step_unpipelined():
        pipeline.input.copy_(host_c, non_blocking=True)
        pipeline.mat1.copy_(host_a, non_blocking=True)
        pipeline.mat2.copy_(host_b, non_blocking=True)
        addmm_kernel(pipeline.input, pipeline.mat1, pipeline.mat2, 1.0, 1.0, pipeline.out)
        host_out.copy_(pipeline.out, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_results = {}
    for name, fn in (("unpipelined", e2e_step_unpipelined), ("pipelined", e2e_step)):
        for _ in range(2):
            fn()
        barrier()
        start.record()
        for _ in range(e2e_steps):
            fn()
        end.record()
        barrier()
        e2e_results[name] = max_over_ranks(start.elapsed_time(end))
    e2e_ms = e2e_results["pipelined"]
    e2e_value = e2e_steps * FLOPS / (e2e_ms * 1e-3) / 1e12
    e2e_unpipelined_value = e2e_steps * FLOPS / (e2e_results["unpipelined"] * 1e-3) / 1e12
    e2e_matches = bool(torch.allclose(host_out.to(device).float(), out.float(), rtol=1e-2, atol=1e-2))
    del host_c, host_a, host_b, pipeline

    # ---- the other kernels of the metric ---------------------------------------
    ops = bench_other_ops(torch, dist, _capi, sharding, device, rank, world, barrier, max_over_ranks)

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        timed_seconds = total_ms * 1e-3
        burst = timed_seconds < 1.0
        peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
        achieved = (FLOPS / world) / (kernel_ms * 1e-3) / 1e12
        line = {
            "metric": "fp16 addmm TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {
                "workload": f"addmm fp16 M=N=K={SIZE}, alpha=beta=1, N(0,1) inputs seed 1",
                "parallelism": "single GPU" if world == 1 else
                               f"N-columns over {world} ranks, A replicated, B and C column slabs, no collective on the "
                               "data path (outputs stay sharded); the step with the slabs all-gathered is reported "
                               "beside it, fused into the epilogue and through NCCL",
                "l2": "inputs (4 x 128 MiB) exceed the 126 MB L2; no flush between steps",
            },
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "gpu_launches_per_step": len(range(0, SIZE, 1024)),
                    "how": "make() handle on 1024-row blocks, copies on two more streams",
                    "unpipelined_value": e2e_unpipelined_value, "matches_device_resident_result": e2e_matches},
            "gpu_launches": args.steps,
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES["gemm_8192"] if world == 1 else None,
                "kernel": "gemm_kernel (tcgen05 cta_group::2, 256x256x64 tiles per CTA pair)", "kernel_ms": kernel_ms,
                "peak_kind": f"{peak_kind} {'burst' if burst else 'sustained'} bf16 cuBLAS",
                "frac_of_spec_2250": achieved / 2250.0,
            },
            "clocks": clocks.summary(),
            "sustained": {"value": sustained_value, "unit": "TFLOP/s", "launches": sustained_launches,
                          "seconds": sustained_ms * 1e-3, "clocks": sustained_clocks.summary(),
                          "frac_of_sustained_peak": sustained_value / world / peaks["bf16_tflops_sustained"]},
            "device_status": status,
            "ops": ops,
        }
        if fused_value is not None:
            line["value_with_fused_all_gather"] = fused_value
            line["value_with_nccl_all_gather"] = nccl_value
            line["fused_all_gather_matches_nccl"] = fused_matches_nccl
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), file=_RESULT_STREAM, flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_other_ops(torch, dist, _capi, sharding, device, rank, world, barrier, max_over_ranks, iters=10):
    """softmax / attention / conv2d / max_pool2d at their benchmark shapes, sharded over the ranks."""
    peaks, _ = measured_peaks()
    results = {}

    def timed(fn):
        for _ in range(3):
            fn()
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        end.record()
        barrier()
        return max_over_ranks(start.elapsed_time(end)) / iters

    gen = torch.Generator(device=device).manual_seed(2 + rank)
    try:
        rows = 65536 // world
        x = (4 * torch.randn(rows, 8192, generator=gen, device=device, dtype=torch.float32)).half()
        y = torch.empty_like(x)
        ms = timed(lambda: _capi.softmax(x, y))
        gbs = 2.0 * 65536 * 8192 * 2 / (ms * 1e-3) / 1e9
        results["softmax_65536x8192_fp16"] = {
            "value": gbs, "unit": "GB/s", "ms": ms, "frac_of_measured_hbm": gbs / (peaks["hbm_gbs"] * world),
            "frac_of_spec_8000": gbs / (8000.0 * world), "sharding": "rows, not gathered"}
        del x, y
    except _capi.KernelLaunchError as error:
        results["softmax_65536x8192_fp16"] = {"error": str(error)}

    try:
        pairs = 128 // world
        q, k, v = (torch.randn(pairs, 1, 4096, 128, generator=gen, device=device, dtype=torch.float32).half()
                   for _ in range(3))
        o = torch.empty_like(q)
        scale = 1.0 / math.sqrt(128)
        for causal in (False, True):
            ms = timed(lambda: _capi.attention(q, k, v, causal, o, scale=scale))
            flops = 4.0 * 128 * 4096 * 4096 * 128 / (2 if causal else 1)
            tf = flops / (ms * 1e-3) / 1e12
            results["attention_b4_h32_s4096_d128" + ("_causal" if causal else "")] = {
                "value": tf, "unit": "TFLOP/s", "ms": ms, "frac_of_measured_bf16": tf / (peaks["bf16_tflops"] * world),
                "frac_of_spec_2250": tf / (2250.0 * world), "sharding": "batch x head, outputs left sharded"}
        del q, k, v, o
    except _capi.KernelLaunchError as error:
        results["attention_b4_h32_s4096_d128"] = {"error": str(error)}

    try:
        batch = 64 // world
        x = torch.randn(batch, 256, 56, 56, generator=gen, device=device, dtype=torch.float32).half()
        w = (torch.randn(256, 256, 3, 3, generator=gen, device=device, dtype=torch.float32) / math.sqrt(2304)).half()
        y = torch.empty(batch, 256, 56, 56, dtype=torch.float16, device=device)
        workspace = torch.empty(max(_capi.conv2d_workspace_size(x, w), 1), dtype=torch.uint8, device=device)
        ms = timed(lambda: _capi.conv2d(x, w, y, 1, 1, workspace=workspace))
        flops = 2.0 * 64 * 56 * 56 * 256 * 2304
        tf = flops / (ms * 1e-3) / 1e12
        results["conv2d_64x256x56x56_k256_3x3"] = {
            "value": tf, "unit": "TFLOP/s", "ms": ms, "frac_of_measured_bf16": tf / (peaks["bf16_tflops"] * world),
            "frac_of_spec_2250": tf / (2250.0 * world), "sharding": "batch, outputs left sharded"}
        # the same problem on channels-last tensors (input, filter and output, as in a channels-last model): x and w
        # are read where they lie, the convolution is a single launch
        x, w, y = (t.contiguous(memory_format=torch.channels_last) for t in (x, w, y))
        ms = timed(lambda: _capi.conv2d(x, w, y, 1, 1, workspace=workspace))
        tf = flops / (ms * 1e-3) / 1e12
        results["conv2d_64x256x56x56_k256_3x3_channels_last"] = {
            "value": tf, "unit": "TFLOP/s", "ms": ms, "frac_of_measured_bf16": tf / (peaks["bf16_tflops"] * world),
            "frac_of_spec_2250": tf / (2250.0 * world), "sharding": "batch, outputs left sharded"}
        del x, w, y
    except _capi.KernelLaunchError as error:
        results["conv2d_64x256x56x56_k256_3x3"] = {"error": str(error)}

    if hasattr(torch, "float8_e5m2"):
        try:
            # 8-bit e5m2 operands, fp16 output (the reference's 8-bit matmul test, at the headline size);
            # rhs as a transposed view, N-columns split over the ranks
            width = SIZE // world
            lhs = torch.randn(SIZE, SIZE, generator=gen, device=device, dtype=torch.float32).to(torch.float8_e5m2)
            rhs = torch.randn(width, SIZE, generator=gen, device=device, dtype=torch.float32).to(torch.float8_e5m2).T
            out8 = torch.empty(SIZE, width, dtype=torch.float16, device=device)
            ms = timed(lambda: _capi.matmul(lhs, rhs, out8))
            tf = FLOPS / (ms * 1e-3) / 1e12
            results["matmul_e5m2_8192"] = {
                "value": tf, "unit": "TFLOP/s", "ms": ms, "frac_of_spec_4500_fp8": tf / (4500.0 * world),
                "sharding": "N-columns, outputs left sharded"}
            del lhs, rhs, out8
        except _capi.KernelLaunchError as error:
            results["matmul_e5m2_8192"] = {"error": str(error)}

    if world == 1:
        try:
            # few output tiles, long reduction: 8 tiles for 148 SMs, so the launcher cuts the reduction over the
            # SMs and a second kernel adds the partial accumulators (32 MB of operands stay in L2 between steps)
            lhs = torch.randn(512, 16384, generator=gen, device=device, dtype=torch.float32).half()
            rhs = torch.randn(16384, 512, generator=gen, device=device, dtype=torch.float32).half()
            small = torch.empty(512, 512, dtype=torch.float16, device=device)
            ms = timed(lambda: _capi.matmul(lhs, rhs, small))
            tf = 2.0 * 512 * 512 * 16384 / (ms * 1e-3) / 1e12
            results["matmul_512x512x16384_split_k"] = {
                "value": tf, "unit": "TFLOP/s", "ms": ms, "launches_per_step": 2,
                "note": "includes the host's launch cost: a step is two launches of ~10 us of device work"}
            del lhs, rhs, small
        except _capi.KernelLaunchError as error:
            results["matmul_512x512x16384_split_k"] = {"error": str(error)}

    try:
        batch = 64 // world
        x = torch.randn(batch, 256, 112, 112, generator=gen, device=device, dtype=torch.float32).half()
        y = torch.empty(batch, 256, 56, 56, dtype=torch.float16, device=device)
        ms = timed(lambda: _capi.max_pool2d(x, y, 2, 2, False))
        moved = (64 * 256 * 112 * 112 + 64 * 256 * 56 * 56) * 2  # every input element read, every output written
        gbs = moved / (ms * 1e-3) / 1e9
        results["max_pool2d_64x256x112x112_2x2"] = {
            "value": gbs, "unit": "GB/s", "ms": ms, "frac_of_measured_hbm": gbs / (peaks["hbm_gbs"] * world),
            "frac_of_spec_8000": gbs / (8000.0 * world), "sharding": "batch, outputs left sharded"}
        del x, y
    except _capi.KernelLaunchError as error:
        results["max_pool2d_64x256x112x112_2x2"] = {"error": str(error)}
    return results


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the host-core baseline leg")
    parser.add_argument("--no-sustained", action="store_true",
                        help="skip the one-second back-to-back window (for short profiler captures)")
    args = parser.parse_args()
    # The contract is ONE line on stdout.  Libraries print there too (NCCL announces its version from C
    # code on the first collective), so everything but the result line is sent to stderr: file
    # descriptor 1 is pointed at stderr for the run and the result goes to a copy of the original.
    global _RESULT_STREAM
    sys.stdout.flush()
    _RESULT_STREAM = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
