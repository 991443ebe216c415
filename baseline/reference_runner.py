"""Runs the UNMODIFIED reference (``baseline/_ref/ninetoothed``) on the definitions in ``examples/``.

Two uses, neither on the product path:

* on a GPU: the reference compiles the definitions to Triton kernels; the parity test
  (``tests/test_reference_parity_gpu.py``) feeds them and this library's kernels the same
  device tensors, and ``bench.py`` times them as the bar to beat (key ``reference_gpu``);
* on the host cores: the same kernels under Triton's interpreter (``TRITON_INTERPRET=1``),
  which is the reference's own CPU path; ``bench.py`` times the README matmul that way.
  Run as a script, this file is that CPU leg (a process of its own, because the
  interpreter switch and the two shims below are process-wide):

      python baseline/reference_runner.py interpret-matmul --size 512 --block 64 --repeat 3

Nothing of the reference is edited.  Two harness-side shims are installed in interpreter
mode only: a stand-in Triton driver when the host has no GPU (the reference asks the
active driver for shared-memory limits even when interpreting, src/ninetoothed/utils.py:5-6
in the reference project), and a fix-up for string annotations in the interpreter's
constexpr detection (Triton 3.6).
"""

from __future__ import annotations

import functools
import json
import os
import pathlib
import sys
import time

ROOT = pathlib.Path(__file__).resolve().parent.parent
REF_DIR = ROOT / "baseline" / "_ref"


def available() -> bool:
    return (REF_DIR / "ninetoothed" / "__init__.py").exists()


def _install_interpreter_shims():
    import torch
    import triton
    import triton.runtime.jit as triton_jit

    class _Utils:
        def get_device_properties(self, device):
            return {"max_shared_mem": 232448, "max_num_regs": 65536, "multiprocessor_count": 148, "warpSize": 32}

    class _StandInDriver:
        utils = _Utils()

        def get_current_device(self):
            return 0

        def get_current_target(self):
            from triton.backends.compiler import GPUTarget

            return GPUTarget("cuda", 100, 32)

        def get_benchmarker(self):
            return lambda fn, quantiles=None, **kw: (fn(), [1.0, 1.0, 1.0])[1]

        def get_device_interface(self):
            return torch.cuda

        def get_active_torch_device(self):
            return torch.device("cpu")

    try:
        triton.runtime.driver.active.get_current_device()
    except Exception:
        triton.runtime.driver.set_active(_StandInDriver())

    normalize = triton_jit._normalize_ty
    if getattr(normalize, "_accepts_strings", False):
        return

    def normalize_with_strings(ty):
        if isinstance(ty, str) and ty.strip().endswith(".constexpr"):
            return "constexpr"
        return normalize(ty)

    normalize_with_strings._accepts_strings = True
    triton_jit._normalize_ty = normalize_with_strings


@functools.lru_cache(maxsize=None)
def definitions(interpret: bool = False):
    """``examples/definitions.py`` executed against the reference package."""
    if not available():
        raise RuntimeError(f"the reference is not installed under {REF_DIR}: run baseline/install_reference.py")
    if interpret:
        os.environ["TRITON_INTERPRET"] = "1"
    elif os.environ.get("TRITON_INTERPRET") == "1":
        raise RuntimeError("TRITON_INTERPRET=1 is set: the compiled reference kernels need a process without it")
    for path in (str(ROOT), str(REF_DIR)):
        if path not in sys.path:
            sys.path.insert(0, path)
    if interpret:
        _install_interpreter_shims()
    import ninetoothed

    if pathlib.Path(ninetoothed.__file__).resolve().parent.parent != REF_DIR.resolve():
        raise RuntimeError(f"'ninetoothed' resolved to {ninetoothed.__file__}, not to the copy under {REF_DIR}")
    from examples import load_definitions

    return load_definitions("ninetoothed")


# ----------------------------------------------------------------------------------------------
# Kernel handles.  `blocks` fixes the block sizes (one configuration, nothing is tuned, as the
# reference's README does by rebinding its block-size names); without it the reference's own
# auto-tuner searches its stock space, capped by `max_num_configs` (src/ninetoothed/make.py:7-17).
# ----------------------------------------------------------------------------------------------
def _tensor(kd, *args, **kwargs):
    return kd.Tensor(*args, **kwargs)


def matmul(blocks=None, interpret=False, application="test", **knobs):
    kd = definitions(interpret)
    arrangement = kd.matmul_arrangement
    if blocks is not None:
        arrangement = functools.partial(arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1],
                                        BLOCK_SIZE_K=blocks[2])
    body = kd.readme_matmul_application if application == "readme" else kd.matmul_application
    return kd.ninetoothed.make(arrangement, body, tuple(kd.Tensor(2) for _ in range(3)), **knobs)


def addmm(blocks=None, interpret=False, **knobs):
    kd = definitions(interpret)
    arrangement = kd.addmm_arrangement
    if blocks is not None:
        arrangement = functools.partial(arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1],
                                        BLOCK_SIZE_K=blocks[2])
    tensors = (kd.Tensor(2), kd.Tensor(2), kd.Tensor(2), kd.Tensor(0), kd.Tensor(0), kd.Tensor(2))
    return kd.ninetoothed.make(arrangement, kd.addmm_application, tensors, **knobs)


def softmax(interpret=False):
    """The row softmax with the row widened to fp32 before exp (what a 16-bit row needs in Triton)."""
    return definitions(interpret).make_softmax_fp32_math()


def scaled_attention(blocks=None, interpret=False, **knobs):
    """The reference's attention body with a scalar ``scale`` folded into the pre-scale of q."""
    kd = definitions(interpret)
    arrangement = kd.scaled_attention_arrangement
    if blocks is not None:
        def arrangement(q, k, v, scale, is_causal, o):
            q_, k_, v_, causal, o_ = kd.attention_arrangement(q, k, v, is_causal, o, BLOCK_SIZE_M=blocks[0],
                                                              BLOCK_SIZE_N=blocks[1])
            return q_, k_, v_, scale, causal, o_
    t = kd._attention_tensor
    tensors = (t(), t(), t(), kd.Tensor(0), kd.Tensor(0, constexpr=True), t())
    return kd.ninetoothed.make(arrangement, kd.scaled_attention_application, tensors, **knobs)


def attention(blocks=None, interpret=False, **knobs):
    """tests/test_attention.py:14-96 of the reference project as it stands (no scale)."""
    kd = definitions(interpret)
    arrangement = kd.attention_arrangement
    if blocks is not None:
        arrangement = functools.partial(arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1])
    t = kd._attention_tensor
    tensors = (t(), t(), t(), kd.Tensor(0, constexpr=True), t())
    return kd.ninetoothed.make(arrangement, kd.attention_application, tensors, **knobs)


def plain_softmax(interpret=False):
    """tests/test_softmax.py:10-27 of the reference project as it stands (fp32 rows)."""
    return definitions(interpret).make_softmax()


def conv2d(blocks=None, interpret=False, **knobs):
    kd = definitions(interpret)
    arrangement = functools.partial(kd.conv2d_arrangement, enable_padding=True)
    if blocks is not None:
        arrangement = functools.partial(arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1],
                                        BLOCK_SIZE_K=blocks[2])
    tensors = (kd.Tensor(4), kd.Tensor(4, shape_options={"constexpr": True}), kd.Tensor(4))
    return kd.ninetoothed.make(arrangement, kd.matmul_application, tensors, **knobs)


def bmm(blocks=None, interpret=False, **knobs):
    """A batch of matmuls on 3-D operands (the matmul body on the batched arrangement of examples/definitions.py)."""
    kd = definitions(interpret)
    arrangement = kd.bmm_arrangement
    if blocks is not None:
        arrangement = functools.partial(arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1],
                                        BLOCK_SIZE_K=blocks[2])
    return kd.ninetoothed.make(arrangement, kd.matmul_application, tuple(kd.Tensor(3) for _ in range(3)), **knobs)


def max_pool2d(ceil_mode=False, interpret=False):
    """tests/test_max_pool2d.py:13-36 of the reference project (its one meta block size is left to its auto-tuner)."""
    return definitions(interpret).make_max_pool2d(ceil_mode)


def best_config(handle):
    """The configuration the reference's auto-tuner settled on (after the first call), as text."""
    kernel = getattr(handle, "_kernel", None)
    config = getattr(kernel, "best_config", None)
    return str(config) if config is not None else None


# ----------------------------------------------------------------------------------------------
# CPU leg: the README matmul (README.md:40-67 in the reference project) under the interpreter
# ----------------------------------------------------------------------------------------------
def _readme_inputs(size: int, rows: int, seed: int):
    import torch

    generator = torch.Generator().manual_seed(seed)
    lhs = torch.randn(size, size, generator=generator).to(torch.float16)
    rhs = torch.randn(size, size, generator=generator).to(torch.float16)
    return lhs[:rows].contiguous(), rhs


def interpret_matmul_step(size: int, block: int, rows: int, seed: int = 0):
    """A callable that runs the README matmul on the first ``rows`` rows of configuration 1 (a bounded sample)."""
    import torch

    kernel = matmul(blocks=(block, block, block), interpret=True, application="readme")
    lhs, rhs = _readme_inputs(size, rows, seed)
    out = torch.empty(rows, size, dtype=torch.float16)
    return lambda: kernel(lhs, rhs, out)


def interpret_matmul(size: int, block: int, repeat: int, rows: int | None = None, seed: int = 0) -> dict:
    import numpy as np
    import torch

    rows = size if rows is None else rows
    kernel = matmul(blocks=(block, block, block), interpret=True, application="readme")
    lhs, rhs = _readme_inputs(size, rows, seed)
    out = torch.empty(rows, size, dtype=torch.float16)
    seconds = []
    for _ in range(repeat):
        start = time.perf_counter()
        kernel(lhs, rhs, out)
        seconds.append(time.perf_counter() - start)
    expected = lhs.float() @ rhs.float()
    error = float((out.float() - expected).abs().max())
    return {
        "workload": f"README matmul {rows} x {size} x {size} fp16, blocks {block}^3, seed {seed}, TRITON_INTERPRET=1",
        "seconds": seconds,
        "median_seconds": float(np.median(seconds)),
        "flop": 2.0 * rows * size * size,
        "max_abs_error_vs_fp32": error,
        "torch_threads": torch.get_num_threads(),
        "cpu_count": os.cpu_count(),
    }


if __name__ == "__main__":
    import argparse

    parser = argparse.ArgumentParser()
    parser.add_argument("leg", choices=["interpret-matmul"])
    parser.add_argument("--size", type=int, default=512)
    parser.add_argument("--block", type=int, default=64)
    parser.add_argument("--repeat", type=int, default=3)
    parser.add_argument("--rows", type=int, default=None, help="only the first ROWS rows of the output (a bounded sample)")
    args = parser.parse_args()
    print(json.dumps(interpret_matmul(args.size, args.block, args.repeat, rows=args.rows)))
