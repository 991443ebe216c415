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
  cpu_baseline  the reference's own CPU path (its README matmul under Triton's
             interpreter), torch.addmm on the host cores, and the numpy port
  ops        the other kernels of the metric (softmax GB/s, attention and conv2d
             TFLOP/s) at their benchmark shapes, sharded over the same ranks, each
             with its own roofline and clock record
  reference_gpu / context  (one GPU) the reference's Triton kernels and torch's library
             operators timed on the same tensors: the bar, not the product

`--impl reference` times the reference's CPU path on the host cores instead (a bounded
sample of its README matmul per step); only rank 0 works.
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
NCU_TRAFFIC_BYTES = {"gemm_8192": 1196186880 + 126215168}  # profiles/gemm_raster_dram.md, the default raster
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
# CPU arm: the reference's own CPU path, torch on the host cores, and the numpy port
# ----------------------------------------------------------------------------
README_MATMUL = {"size": 512, "block": 64}  # configuration 1 of the benchmark (README.md:40-67 in the reference project)


def usable_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU legs set the thread
    counts themselves so that the baseline does not depend on how the process was launched."""
    import torch

    cores = usable_cores()
    torch.set_num_threads(cores)
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=cores)
    except Exception:
        pass
    return cores


def blas_threads():
    try:
        from threadpoolctl import threadpool_info

        counts = [pool.get("num_threads", 1) for pool in threadpool_info() if pool.get("user_api") == "blas"]
        return max(counts) if counts else None
    except Exception:
        return None


def spread(samples):
    return (max(samples) - min(samples)) / statistics.median(samples) if len(samples) > 1 else 0.0


def interpreter_matmul_leg(size=README_MATMUL["size"], block=README_MATMUL["block"], repeat=1, rows=None):
    """The reference's README matmul under TRITON_INTERPRET=1 in a process of its own (the switch is
    process-wide).  None when the reference is not installed under baseline/_ref."""
    from baseline import reference_runner

    if not reference_runner.available():
        return None
    command = [sys.executable, str(ROOT / "baseline" / "reference_runner.py"), "interpret-matmul", "--size", str(size),
               "--block", str(block), "--repeat", str(repeat)]
    if rows is not None:
        command += ["--rows", str(rows)]
    env = dict(os.environ, OMP_NUM_THREADS=str(usable_cores()), CUDA_VISIBLE_DEVICES="")
    done = subprocess.run(command, capture_output=True, text=True, env=env)
    if done.returncode != 0:
        return {"error": (done.stderr.strip().splitlines() or ["failed"])[-1][:300]}
    return json.loads(done.stdout.strip().splitlines()[-1])


def torch_cpu_addmm_leg(n=SIZE, runs=3):
    """torch.addmm on the host cores at the headline shape, fp32 (torch's CPU GEMM of fp16 is not a tuned path)."""
    import torch

    generator = torch.Generator().manual_seed(1)
    c, a, b = (torch.randn(n, n, generator=generator, dtype=torch.float32) for _ in range(3))
    out = torch.empty(n, n, dtype=torch.float32)
    torch.addmm(c, a, b, out=out)  # warm-up: thread pool, pages
    seconds = []
    for _ in range(runs):
        t0 = time.perf_counter()
        torch.addmm(c, a, b, out=out)
        seconds.append(time.perf_counter() - t0)
    median = statistics.median(seconds)
    return {"value": 2.0 * n**3 / median / 1e12, "unit": "TFLOP/s", "median_seconds": median, "runs": runs,
            "spread": spread(seconds), "dtype": "f32", "threads": torch.get_num_threads(),
            "workload": f"torch.addmm fp32 {n}^3 on the host cores"}


def numpy_port_leg(n=2048, runs=3):
    """oracle.kernels.addmm: the numpy restatement of the reference's tiled loop (fp16 in, fp32 accumulate)."""
    import numpy as np

    from oracle import inputs as oi
    from oracle import kernels as ok

    c, a, b = oi.addmm_inputs(n, n, n, 1)
    block = min(n, 1024)
    seconds = []
    for _ in range(runs):
        t0 = time.perf_counter()
        ok.addmm(c, a, b, 1.0, 1.0, np.float16, block, block, block)
        seconds.append(time.perf_counter() - t0)
    median = statistics.median(seconds)
    return {"value": 2.0 * n**3 / median / 1e12, "unit": "TFLOP/s", "median_seconds": median, "runs": runs,
            "spread": spread(seconds), "blas_threads": blas_threads(),
            "workload": f"oracle.kernels.addmm (numpy) on {n}^3 fp16"}


def cpu_baseline():
    """The host-core figures printed beside the GPU number: (i) the reference's own CPU path, i.e. its README
    matmul (512^3, 64^3 blocks, seed 0) under Triton's interpreter, once; (ii) torch.addmm on all host
    cores at the headline shape; (iii) the numpy port.  `value` is (i) when the reference is installed."""
    cores = use_all_host_threads()
    legs = {"torch_cpu": torch_cpu_addmm_leg(), "numpy_port": numpy_port_leg()}
    interpreted = interpreter_matmul_leg()
    if interpreted is not None and "error" not in interpreted:
        value = interpreted["flop"] / interpreted["median_seconds"] / 1e12
        legs["interpreter"] = {"value": value, "unit": "TFLOP/s", "seconds": interpreted["seconds"],
                               "max_abs_error_vs_fp32": interpreted["max_abs_error_vs_fp32"]}
        return {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "reference",
                "sample": f"{interpreted['workload']}: the whole of configuration 1, one run of "
                          f"{interpreted['median_seconds']:.1f} s (a single Python thread drives the interpreter; "
                          f"numpy inside it may use {cores} threads); rate = 2*512^3 FLOP / that time",
                "os_cpu_count": os.cpu_count(), **legs}
    port = legs["numpy_port"]
    return {"value": port["value"], "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": port["workload"] + (f"; the reference's interpreter leg failed: {interpreted['error']}"
                                          if interpreted else "; the reference is not installed under baseline/_ref"),
            "os_cpu_count": os.cpu_count(), **legs}


def run_reference(args):
    """--impl reference: the reference's own CPU path for the headline kind of work (a tiled fp16 matmul with
    fp32 accumulation), timed on the host cores.  A step is a BOUNDED SAMPLE of configuration 1: the first 64
    rows of output tiles of the README matmul (64 x 512 x 512, 64^3 blocks) under Triton's interpreter, about
    a second, so that warm-up plus steps stay within a few minutes; rates are FLOP-normalised.  The whole
    of configuration 1 (once) and torch.addmm at the 8192^3 shape are reported in `cpu_baseline`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = use_all_host_threads()
    from baseline import reference_runner

    size, block, rows = README_MATMUL["size"], README_MATMUL["block"], 64
    if reference_runner.available():
        os.environ["CUDA_VISIBLE_DEVICES"] = ""
        step = reference_runner.interpret_matmul_step(size, block, rows)
        kind = "reference"
        sample = (f"README matmul under TRITON_INTERPRET=1, {rows} x {size} x {size} of configuration 1 per step "
                  f"(blocks {block}^3, seed 0)")
        flop = 2.0 * rows * size * size
    else:
        import numpy as np

        from oracle import inputs as oi
        from oracle import kernels as ok

        c, a, b = oi.addmm_inputs(2048, 2048, 2048, 1)
        step = lambda: ok.addmm(c, a, b, 1.0, 1.0, np.float16, 1024, 1024, 1024)  # noqa: E731
        kind = "port"
        sample = "oracle.kernels.addmm (numpy port) on 2048^3 per step; the reference is not installed under baseline/_ref"
        flop = 2.0 * 2048**3
    for _ in range(args.warmup):
        step()
    seconds = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        step()
        seconds.append(time.perf_counter() - t0)
    elapsed = sum(seconds)
    value = args.steps * flop / elapsed / 1e12
    whole = interpreter_matmul_leg() if kind == "reference" else None
    line = {
        "impl": "reference", "metric": "fp16 addmm TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"addmm fp16 M=N=K={SIZE}, alpha=beta=1 (the reference's CPU path cannot run that "
                               f"shape: each step is a bounded sample, {sample}; FLOP-normalised)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample,
                         "spread": spread(seconds), "os_cpu_count": os.cpu_count(),
                         "whole_configuration_1": whole, "torch_cpu": torch_cpu_addmm_leg()},
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
    # the other way of making the copies (peer stores when the default goes through the switch, and the reverse
    # where a multicast mapping exists), timed beside the default
    other_gathered = None
    if world > 1 and gathered.multicast_slab_ptr:
        other_gathered = sharding.GatheredColumns(SIZE, SIZE, torch.float16, device,
                                                  through_switch=not gathered.through_switch)
    fused_matches_nccl = other_matches_nccl = None
    if world > 1:
        _capi.addmm(c_in, a, b, 1.0, 1.0, out)
        unfused = sharding.gather_columns(out)
        gathered.addmm(c_in, a, b, 1.0, 1.0)
        fused_matches_nccl = bool(torch.equal(gathered.wait(), unfused))
        if other_gathered is not None:
            other_gathered.addmm(c_in, a, b, 1.0, 1.0)
            other_matches_nccl = bool(torch.equal(other_gathered.wait(), unfused))
        del unfused

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

    if args.headline_only:
        # For profiler captures of the dominant kernel: the headline launches and nothing else.
        if rank == 0:
            print(json.dumps({"metric": "fp16 addmm TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                              "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
                              "kernel_ms": kernel_ms, "device_status": status, "clocks": clocks.summary(),
                              "config": {"workload": f"addmm fp16 M=N=K={SIZE}, alpha=beta=1, N(0,1) inputs seed 1",
                                         "note": "--headline-only: no end-to-end leg, no other kernels, no baselines"}}),
                  file=_RESULT_STREAM, flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- for N > 1: the same step with the column slabs reassembled on every rank, two ways -----
    fused_value = nccl_value = other_fused_value = None
    if world > 1:
        barrier()
        start.record()
        for _ in range(args.steps):
            gathered.addmm(c_in, a, b, 1.0, 1.0)
            gathered.wait()
        end.record()
        barrier()
        fused_value = args.steps * FLOPS / (max_over_ranks(start.elapsed_time(end)) * 1e-3) / 1e12
        if other_gathered is not None:
            barrier()
            start.record()
            for _ in range(args.steps):
                other_gathered.addmm(c_in, a, b, 1.0, 1.0)
                other_gathered.wait()
            end.record()
            barrier()
            other_fused_value = args.steps * FLOPS / (max_over_ranks(start.elapsed_time(end)) * 1e-3) / 1e12
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
    # the plain sequence copy-in, one call, copy-out is timed beside it.  With several ranks every
    # rank brings in only its rows of the replicated mat1 and the ranks all-gather it over NVLink.
    from ninetoothed_b200.host_pipeline import HostAddmm, ShardedHostAddmm

    host_c, host_b = (t.cpu().pin_memory() for t in (c_in, b))
    host_out = torch.empty(SIZE, width, dtype=torch.float16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    e2e_results = {}
    if world == 1:
        host_a = a.cpu().pin_memory()
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

        # The same pipeline with consecutive steps allowed to overlap: a step's copies in wait for the previous step's
        # kernels only, so one step's last kernel and copy out run under the next step's copies in; the caller joins
        # the copies out once, at the end (inside the timed region).
        overlapped = HostAddmm(addmm_kernel, SIZE, width, SIZE, torch.float16, device, row_block=1024,
                               overlap_steps=True)
        host_out_overlapped = torch.empty_like(host_out).pin_memory()

        def e2e_step_overlapped():
            overlapped(host_c, host_a, host_b, 1.0, 1.0, host_out_overlapped)

        legs = (("unpipelined", e2e_step_unpipelined, None), ("pipelined", e2e_step, None),
                ("overlapped", e2e_step_overlapped, overlapped.wait))
        e2e_how = "make() handle on 1024-row blocks, copies on two more streams"
    else:
        pipeline = ShardedHostAddmm(addmm_kernel, SIZE, width, SIZE, torch.float16, device, row_block=1024)
        host_a = a[pipeline.rows].cpu().pin_memory()  # this rank's rows of the replicated operand
        h2d, d2h = pipeline.h2d_bytes() * world, pipeline.d2h_bytes() * world  # whole job, like `value`
        overlapped = ShardedHostAddmm(addmm_kernel, SIZE, width, SIZE, torch.float16, device, row_block=1024,
                                      overlap_steps=True)
        host_out_overlapped = torch.empty_like(host_out).pin_memory()

        def e2e_step():
            pipeline(host_c, host_a, host_b, 1.0, 1.0, host_out)

        def e2e_step_overlapped():
            overlapped(host_c, host_a, host_b, 1.0, 1.0, host_out_overlapped)

        legs = (("pipelined", e2e_step, None), ("overlapped", e2e_step_overlapped, overlapped.wait))
        e2e_how = ("make() handle on 1024-row blocks, copies on two more streams; each rank copies in 1/N of the "
                   "rows of mat1 and the ranks all-gather it over NVLink (NCCL); bytes are whole-job sums")
    for name, fn, finish in legs:
        for _ in range(2):
            fn()
        if finish is not None:
            finish()
        barrier()
        start.record()
        for _ in range(e2e_steps):
            fn()
        if finish is not None:
            finish()  # the caller's stream joins the copies out: every step's result is in host memory at `end`
        end.record()
        barrier()
        e2e_results[name] = max_over_ranks(start.elapsed_time(end))
    e2e_per_call_join_value = e2e_steps * FLOPS / (e2e_results["pipelined"] * 1e-3) / 1e12
    e2e_ms = e2e_results["pipelined"]
    if "overlapped" in e2e_results:
        overlapped_ok = bool(torch.allclose(host_out_overlapped.to(device).float(), out.float(), rtol=1e-2, atol=1e-2))
        if world > 1:  # every rank must take the same leg
            verdict = torch.tensor([1 if overlapped_ok else 0], device=device)
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
            overlapped_ok = bool(verdict.item())
        if overlapped_ok and e2e_results["overlapped"] < e2e_ms:
            e2e_ms = e2e_results["overlapped"]
            e2e_how += ("; consecutive steps overlap (a step's copies in wait for the previous step's kernels only, "
                        "the copies out are joined once at the end of the timed region)")
        del overlapped, host_out_overlapped
    e2e_value = e2e_steps * FLOPS / (e2e_ms * 1e-3) / 1e12
    e2e_unpipelined_value = (e2e_steps * FLOPS / (e2e_results["unpipelined"] * 1e-3) / 1e12
                             if "unpipelined" in e2e_results else None)
    e2e_matches = bool(torch.allclose(host_out.to(device).float(), out.float(), rtol=1e-2, atol=1e-2))
    if world > 1:
        flag = torch.tensor([1 if e2e_matches else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        e2e_matches = bool(flag.item())
    del host_c, host_a, host_b, pipeline

    # ---- one GPU: the reference's own Triton kernel and torch's library GEMM on the same tensors ----
    reference, reference_gpu, context = None, {}, {}
    if world == 1 and not args.no_reference_gpu:
        from baseline import reference_runner

        timer = OpTimer(torch, device.index, barrier, max_over_ranks)
        scratch = torch.empty_like(out)
        ms, iters, _ = timer(lambda: torch.addmm(c_in, a, b, out=scratch), min_iters=20, min_ms=15.0, clocks=False)
        context["torch.addmm"] = {"ms": ms, "value": FLOPS / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "iters": iters}
        if reference_runner.available():
            reference = reference_runner
            try:
                kernel = reference.addmm(blocks=(128, 256, 64), num_warps=8, num_stages=4)
                kernel(c_in, a, b, 1.0, 1.0, scratch)
                ms, iters, _ = timer(lambda: kernel(c_in, a, b, 1.0, 1.0, scratch), min_iters=10, min_ms=15.0,
                                     clocks=False)
                reference_gpu["addmm_8192_fp16"] = {
                    "ms": ms, "value": FLOPS / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "iters": iters,
                    "config": "BLOCK_SIZE_M=128, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, num_warps=8, num_stages=4",
                    "identical_elements": float((scratch == out).float().mean().item())}
            except Exception as error:
                reference_gpu["addmm_8192_fp16"] = {"unavailable": f"{type(error).__name__}: {str(error)[:200]}"}
        del scratch

    # ---- the other kernels of the metric ---------------------------------------
    ops, ops_reference_gpu, ops_context = bench_other_ops(torch, dist, _capi, sharding, device, rank, world, barrier,
                                                          max_over_ranks, reference=reference,
                                                          with_context=not args.no_reference_gpu)
    reference_gpu.update(ops_reference_gpu)
    context.update(ops_context)

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
                               f"N-columns over {world} ranks, A replicated, B and C column slabs. `value` is the step "
                               "with the output column slabs LEFT SHARDED (no collective on the data path); the step "
                               "with the slabs all-gathered onto every rank, as the configuration words it, is "
                               "`value_with_fused_all_gather` (gather fused into the GEMM epilogue) and "
                               "`value_with_nccl_all_gather` (kernel, then NCCL)",
                "l2": "inputs (4 x 128 MiB) exceed the 126 MB L2; no flush between steps",
            },
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "gpu_launches_per_step": len(range(0, SIZE, 1024)) * world,
                    "how": e2e_how,
                    "unpipelined_value": e2e_unpipelined_value, "per_call_join_value": e2e_per_call_join_value,
                    "matches_device_resident_result": e2e_matches},
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
        if world == 1:
            # Not the product: the reference's Triton kernels (fixed block sizes found with its own
            # auto-tuner on a B200, compile time excluded) and torch's library operators, timed in this
            # run on the same tensors.
            line["reference_gpu"] = dict(reference_gpu, how=(
                "unmodified reference from baseline/_ref compiled by Triton on this GPU, definitions of "
                "examples/definitions.py, CUDA events" if reference is not None else
                "unavailable: the reference is not installed under baseline/_ref"))
            line["context"] = dict(context, note="library kernels through torch, for orientation; not the product")
            if "ms" in reference_gpu.get("addmm_8192_fp16", {}):
                line["roofline"]["vs_reference_gpu"] = reference_gpu["addmm_8192_fp16"]["ms"] / kernel_ms
        if fused_value is not None:
            line["value_with_fused_all_gather"] = fused_value
            line["value_with_nccl_all_gather"] = nccl_value
            line["fused_all_gather_matches_nccl"] = fused_matches_nccl
            way = lambda through_switch: ("one multimem.st per 16 bytes, copies made by the NVSwitch"
                                          if through_switch else "a plain store per rank over NVLink")
            line["fused_all_gather"] = {"how": way(gathered.through_switch), "value": fused_value}
            if other_fused_value is not None:
                line["fused_all_gather"]["other_way"] = {"how": way(other_gathered.through_switch),
                                                         "value": other_fused_value,
                                                         "matches_nccl": other_matches_nccl}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), file=_RESULT_STREAM, flush=True)
    if world > 1:
        dist.destroy_process_group()


class OpTimer:
    """Times one kernel for the `ops` table: three warm-up launches, then at least 50 launches and at
    least 20 ms of them (a 0.08 ms kernel gets 250), between CUDA events on the launching stream, max over
    ranks, with the GPU's clock sampled over exactly that region."""

    def __init__(self, torch, device_index, barrier, max_over_ranks):
        self.torch, self.index, self.barrier, self.max_over_ranks = torch, device_index, barrier, max_over_ranks

    def _run(self, fn, iters):
        start, end = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        self.barrier()
        start.record()
        for _ in range(iters):
            fn()
        end.record()
        self.barrier()
        return self.max_over_ranks(start.elapsed_time(end)) / iters

    def __call__(self, fn, min_iters=50, min_ms=20.0, clocks=True):
        for _ in range(3):
            fn()
        estimate = self._run(fn, 5)
        iters = int(min(5000, max(min_iters, math.ceil(min_ms / max(estimate, 1e-4)))))
        if not clocks:
            return self._run(fn, iters), iters, None
        with ClockSampler(self.index) as sampler:
            ms = self._run(fn, iters)
        return ms, iters, sampler.summary()


def op_entry(value, unit, ms, iters, clocks, world, bound, algorithmic, peak, peak_kind, spec, sharding, **more):
    """One row of `ops`, shaped like the headline's roofline: achieved / peak per GPU, the algorithmic work."""
    per_gpu = value / world
    entry = {"value": value, "unit": unit, "ms": ms, "iters": iters, "sharding": sharding,
             "roofline": {"bound": bound, "achieved": per_gpu, "peak": peak, "unit": unit, "frac": per_gpu / peak,
                          "kernel_ms": ms, "peak_kind": peak_kind,
                          ("algorithmic_bytes" if bound == "hbm" else "algorithmic_flop"): algorithmic,
                          "frac_of_spec": per_gpu / spec, "spec": spec},
             "clocks": clocks}
    entry.update(more)
    return entry


def bench_other_ops(torch, dist, _capi, sharding, device, rank, world, barrier, max_over_ranks, reference=None,
                    with_context=True):
    """softmax / attention / conv2d / max_pool2d at their benchmark shapes, sharded over the ranks.

    `reference` (one GPU only): baseline.reference_runner when the reference is installed; its Triton kernels
    are then timed on the same tensors (fixed block sizes, compile excluded) and library operators of torch
    are timed as context.  Neither is the product."""
    import torch.nn.functional as F

    peaks, peak_kind = measured_peaks()
    timer = OpTimer(torch, device.index, barrier, max_over_ranks)
    results, reference_gpu, context = {}, {}, {}
    tensor_peak, hbm_peak = peaks["bf16_tflops"], peaks["hbm_gbs"]
    tensor_kind, hbm_kind = f"{peak_kind} burst bf16 cuBLAS", f"{peak_kind} copy bandwidth"

    def side(table, name, fn, work, unit_scale, **more):
        """Time a comparator (not the product) on the tensors at hand."""
        if not with_context:
            return
        try:
            fn()  # compiles on first use
            ms, iters, _ = timer(fn, min_iters=10, min_ms=10.0, clocks=False)
            table[name] = {"ms": ms, "value": work / (ms * 1e-3) / unit_scale, "iters": iters, **more}
        except Exception as error:  # a comparator that does not build or run is reported, not fatal
            table[name] = {"unavailable": f"{type(error).__name__}: {str(error)[:200]}"}

    gen = torch.Generator(device=device).manual_seed(2 + rank)
    try:
        rows = 65536 // world
        x = (4 * torch.randn(rows, 8192, generator=gen, device=device, dtype=torch.float32)).half()
        y = torch.empty_like(x)
        ms, iters, clocks = timer(lambda: _capi.softmax(x, y))
        moved = 2.0 * 65536 * 8192 * 2
        results["softmax_65536x8192_fp16"] = op_entry(
            moved / (ms * 1e-3) / 1e9, "GB/s", ms, iters, clocks, world, "hbm", moved, hbm_peak, hbm_kind, 8000.0,
            "rows, not gathered")
        if world == 1:
            side(context, "torch.softmax", lambda: torch.softmax(x, -1, out=y), moved, 1e9, unit="GB/s")
            if reference is not None:
                kernel = reference.softmax()
                side(reference_gpu, "softmax_65536x8192_fp16", lambda: kernel(x, y, BLOCK_SIZE=8192), moved, 1e9,
                     unit="GB/s", config="BLOCK_SIZE=8192, row widened to fp32")
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
            name = "attention_b4_h32_s4096_d128" + ("_causal" if causal else "")
            ms, iters, clocks = timer(lambda: _capi.attention(q, k, v, causal, o, scale=scale))
            flops = 4.0 * 128 * 4096 * 4096 * 128 / (2 if causal else 1)
            results[name] = op_entry(flops / (ms * 1e-3) / 1e12, "TFLOP/s", ms, iters, clocks, world, "tensor", flops,
                                     tensor_peak, tensor_kind, 2250.0, "batch x head, outputs left sharded")
            if world == 1:
                side(context, "F.scaled_dot_product_attention" + ("_causal" if causal else ""),
                     lambda: F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale), flops, 1e12,
                     unit="TFLOP/s")
                if reference is not None:
                    kernel = reference.scaled_attention(blocks=(128, 32), num_warps=4, num_stages=3)
                    theirs = torch.empty_like(o)
                    side(reference_gpu, name, lambda: kernel(q, k, v, scale, causal, theirs), flops, 1e12,
                         unit="TFLOP/s", config="BLOCK_SIZE_M=128, BLOCK_SIZE_N=32, num_warps=4, num_stages=3")
                    if "ms" in reference_gpu[name]:
                        fp32 = F.scaled_dot_product_attention(q[:8].float(), k[:8].float(), v[:8].float(),
                                                              is_causal=causal, scale=scale)
                        reference_gpu[name]["max_abs_error_vs_fp32_sdpa"] = float((theirs[:8].float() - fp32).abs().max())
                        reference_gpu[name]["ours_max_abs_error_vs_fp32_sdpa"] = float((o[:8].float() - fp32).abs().max())
                        del fp32
                    del theirs
        del q, k, v, o
    except _capi.KernelLaunchError as error:
        results["attention_b4_h32_s4096_d128"] = {"error": str(error)}

    try:
        batch = 64 // world
        x = torch.randn(batch, 256, 56, 56, generator=gen, device=device, dtype=torch.float32).half()
        w = (torch.randn(256, 256, 3, 3, generator=gen, device=device, dtype=torch.float32) / math.sqrt(2304)).half()
        y = torch.empty(batch, 256, 56, 56, dtype=torch.float16, device=device)
        workspace = torch.empty(max(_capi.conv2d_workspace_size(x, w), 1), dtype=torch.uint8, device=device)
        ms, iters, clocks = timer(lambda: _capi.conv2d(x, w, y, 1, 1, workspace=workspace))
        flops = 2.0 * 64 * 56 * 56 * 256 * 2304
        results["conv2d_64x256x56x56_k256_3x3"] = op_entry(
            flops / (ms * 1e-3) / 1e12, "TFLOP/s", ms, iters, clocks, world, "tensor", flops, tensor_peak, tensor_kind,
            2250.0, "batch, outputs left sharded", launches_per_step=2)
        if world == 1:
            side(context, "F.conv2d", lambda: F.conv2d(x, w, padding=1), flops, 1e12, unit="TFLOP/s")
            if reference is not None:
                kernel = reference.conv2d(blocks=(128, 256, 64), num_warps=8, num_stages=3)
                side(reference_gpu, "conv2d_64x256x56x56_k256_3x3", lambda: kernel(x, w, y, padding_h=1, padding_w=1),
                     flops, 1e12, unit="TFLOP/s",
                     config="BLOCK_SIZE_M=128, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, num_warps=8, num_stages=3")
        # the same problem on channels-last tensors (input, filter and output, as in a channels-last model): x and w
        # are read where they lie, the convolution is a single launch
        x, w, y = (t.contiguous(memory_format=torch.channels_last) for t in (x, w, y))
        ms, iters, clocks = timer(lambda: _capi.conv2d(x, w, y, 1, 1, workspace=workspace))
        results["conv2d_64x256x56x56_k256_3x3_channels_last"] = op_entry(
            flops / (ms * 1e-3) / 1e12, "TFLOP/s", ms, iters, clocks, world, "tensor", flops, tensor_peak, tensor_kind,
            2250.0, "batch, outputs left sharded", launches_per_step=1)
        if world == 1:
            side(context, "F.conv2d_channels_last", lambda: F.conv2d(x, w, padding=1), flops, 1e12, unit="TFLOP/s")
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
            ms, iters, clocks = timer(lambda: _capi.matmul(lhs, rhs, out8))
            results["matmul_e5m2_8192"] = op_entry(
                FLOPS / (ms * 1e-3) / 1e12, "TFLOP/s", ms, iters, clocks, world, "tensor", FLOPS, 2.0 * tensor_peak,
                f"twice the {tensor_kind} (no 8-bit peak was measured)", 4500.0, "N-columns, outputs left sharded")
            del lhs, rhs, out8
        except _capi.KernelLaunchError as error:
            results["matmul_e5m2_8192"] = {"error": str(error)}

    try:
        # a batch of 64 matmuls of 1024^3 (the batched matmul of the reference's build guide), batch split over ranks
        count = 64 // world
        lhs = torch.randn(count, 1024, 1024, generator=gen, device=device, dtype=torch.float32).half()
        rhs = torch.randn(count, 1024, 1024, generator=gen, device=device, dtype=torch.float32).half()
        outb = torch.empty(count, 1024, 1024, dtype=torch.float16, device=device)
        ms, iters, clocks = timer(lambda: _capi.bmm(lhs, rhs, outb))
        flops = 2.0 * 64 * 1024**3
        results["bmm_64x1024x1024x1024"] = op_entry(
            flops / (ms * 1e-3) / 1e12, "TFLOP/s", ms, iters, clocks, world, "tensor", flops, tensor_peak, tensor_kind,
            2250.0, "batch, outputs left sharded")
        if world == 1:
            side(context, "torch.bmm", lambda: torch.bmm(lhs, rhs, out=outb), flops, 1e12, unit="TFLOP/s")
        del lhs, rhs, outb
    except _capi.KernelLaunchError as error:
        results["bmm_64x1024x1024x1024"] = {"error": str(error)}

    if world == 1:
        try:
            # few output tiles, long reduction: 8 tiles for 148 SMs, so the launcher cuts the reduction over the
            # SMs and a second kernel adds the partial accumulators (32 MB of operands stay in L2 between steps)
            lhs = torch.randn(512, 16384, generator=gen, device=device, dtype=torch.float32).half()
            rhs = torch.randn(16384, 512, generator=gen, device=device, dtype=torch.float32).half()
            small = torch.empty(512, 512, dtype=torch.float16, device=device)
            ms, iters, clocks = timer(lambda: _capi.matmul(lhs, rhs, small))
            flops = 2.0 * 512 * 512 * 16384
            results["matmul_512x512x16384_split_k"] = op_entry(
                flops / (ms * 1e-3) / 1e12, "TFLOP/s", ms, iters, clocks, world, "tensor", flops, tensor_peak,
                tensor_kind, 2250.0, "one GPU", launches_per_step=2,
                note="includes the host's launch cost: a step is two launches of ~10 us of device work")
            side(context, "torch.matmul_512x512x16384", lambda: torch.matmul(lhs, rhs, out=small), flops, 1e12,
                 unit="TFLOP/s")
            del lhs, rhs, small
        except _capi.KernelLaunchError as error:
            results["matmul_512x512x16384_split_k"] = {"error": str(error)}

    try:
        batch = 64 // world
        x = torch.randn(batch, 256, 112, 112, generator=gen, device=device, dtype=torch.float32).half()
        y = torch.empty(batch, 256, 56, 56, dtype=torch.float16, device=device)
        ms, iters, clocks = timer(lambda: _capi.max_pool2d(x, y, 2, 2, False))
        moved = (64 * 256 * 112 * 112 + 64 * 256 * 56 * 56) * 2.0  # every input element read, every output written
        results["max_pool2d_64x256x112x112_2x2"] = op_entry(
            moved / (ms * 1e-3) / 1e9, "GB/s", ms, iters, clocks, world, "hbm", moved, hbm_peak, hbm_kind, 8000.0,
            "batch, outputs left sharded")
        if world == 1:
            side(context, "F.max_pool2d", lambda: F.max_pool2d(x, 2), moved, 1e9, unit="GB/s")
        del x, y
    except _capi.KernelLaunchError as error:
        results["max_pool2d_64x256x112x112_2x2"] = {"error": str(error)}
    for name, entry in reference_gpu.items():
        if "ms" in entry and name in results and "ms" in results[name]:
            results[name]["vs_reference_gpu"] = entry["ms"] / results[name]["ms"]
    return results, reference_gpu, context


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the host-core baseline leg")
    parser.add_argument("--no-reference-gpu", action="store_true",
                        help="skip the reference's Triton kernels and the torch library context (one GPU only)")
    parser.add_argument("--headline-only", action="store_true",
                        help="time the headline kernel and stop (for profiler captures of that kernel)")
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
