"""``make(..., caller="cuda")``: files in the reference's ahead-of-time shape (src/ninetoothed/aot.py:18-44,
126-147, 802-862 in the reference project).

CPU part: the header, the source and the library are written, the header carries the launch line the
reference's loader parses, the library exports the symbol, and the reference's OWN loader
(``ninetoothed.aot._load_launch_func`` from ``baseline/_ref``, when installed) accepts the pair.
GPU part: the kernels are run through this library's loader and through the reference's, against the oracle.
"""

import ctypes
import functools
import pathlib
import re
import sys

import numpy as np
import pytest

import ninetoothed_b200 as ninetoothed
from ninetoothed_b200 import Tensor, aot

from examples import definitions as kd

ROOT = pathlib.Path(__file__).resolve().parent.parent


def reference_loader():
    """The reference's ``_load_launch_func`` (unmodified), or None where the reference is not installed."""
    from baseline import reference_runner

    if not reference_runner.available():
        return None
    if str(reference_runner.REF_DIR) not in sys.path:
        sys.path.insert(0, str(reference_runner.REF_DIR))
    try:
        import ninetoothed.aot as reference_aot
    except Exception:  # the reference imports Triton's active driver at import time: no GPU, no loader
        return None
    return reference_aot._load_launch_func


def make_addmm(tmp_path, name="addmm_aot", dtype=ninetoothed.float16, scalar_dtype=None):
    arrangement = functools.partial(kd.addmm_arrangement, BLOCK_SIZE_M=64, BLOCK_SIZE_N=64, BLOCK_SIZE_K=64)
    tensors = tuple(Tensor(ndim, dtype=(dtype if ndim else scalar_dtype)) for ndim in (2, 2, 2, 0, 0, 2))
    return ninetoothed.make(arrangement, kd.addmm_application, tensors, caller="cuda", kernel_name=name,
                            output_dir=tmp_path)


def test_files_have_the_reference_shape(tmp_path):
    kernel = make_addmm(tmp_path)
    assert callable(kernel)
    header = (tmp_path / "addmm_aot.h").read_text()
    match = re.search(r"NineToothedResult\s+launch_addmm_aot\s*\((.*?)\)\s*;", header)
    assert match is not None
    params = [p.strip() for p in match.group(1).split(",")]
    assert params[0] == "NineToothedStream stream"
    assert sum(p.startswith("NineToothedTensor ") for p in params) == 6
    library = ctypes.CDLL(str(tmp_path / "addmm_aot.so"))
    assert library.launch_addmm_aot is not None
    assert (tmp_path / "addmm_aot.cpp").exists()


def test_every_kernel_with_a_fixed_signature_has_an_ahead_of_time_form(tmp_path):
    """The forwarders compile and export their symbol (no GPU needed for that)."""
    f16, bf16 = ninetoothed.float16, ninetoothed.bfloat16
    t4 = lambda dtype=f16: Tensor(4, dtype=dtype)  # noqa: E731
    cases = {
        "matmul_bf16": (kd.matmul_arrangement, kd.matmul_application, tuple(Tensor(2, dtype=bf16) for _ in range(3))),
        "bmm_f16": (kd.bmm_arrangement, kd.matmul_application, tuple(Tensor(3, dtype=f16) for _ in range(3))),
        "attention_causal": (kd.attention_arrangement, kd.attention_application,
                             (t4(), t4(), t4(), Tensor(0, constexpr=True, value=1), t4())),
        "attention_with_scale": (kd.scaled_attention_arrangement, kd.scaled_attention_application,
                             (t4(), t4(), t4(), Tensor(0, dtype=ninetoothed.float32), Tensor(0, constexpr=True, value=0), t4())),
        "conv2d_unpadded": kd.conv2d_premake(dtype=f16),
    }
    for name, (arrangement, application, tensors) in cases.items():
        ninetoothed.make(arrangement, application, tensors, caller="cuda", kernel_name=name, output_dir=tmp_path)
        assert getattr(ctypes.CDLL(str(tmp_path / f"{name}.so")), f"launch_{name}") is not None
        source = (tmp_path / f"{name}.cpp").read_text()
        assert "NINETOOTHED_BFLOAT16" in source if name == "matmul_bf16" else "NINETOOTHED_FLOAT16" in source
    assert "causal_value = 1" in (tmp_path / "attention_causal.cpp").read_text()
    assert "causal_value = 0" in (tmp_path / "attention_with_scale.cpp").read_text()
    with pytest.raises(aot.AotError, match="is taken"):  # would clash with the library's own launch_matmul
        ninetoothed.make(*cases["matmul_bf16"], caller="cuda", kernel_name="matmul", output_dir=tmp_path)
    with pytest.raises(aot.AotError):  # the padded conv2d leaves padding_h / padding_w to the call
        ninetoothed.make(functools.partial(kd.conv2d_arrangement, enable_padding=True), kd.matmul_application,
                         (t4(), Tensor(4, dtype=f16, shape_options={"constexpr": True}), t4()), caller="cuda",
                         kernel_name="conv2d_padded", output_dir=tmp_path)


def test_what_cannot_be_fixed_ahead_of_time_is_rejected(tmp_path):
    with pytest.raises(aot.AotError):  # no dtype on the tensors
        ninetoothed.make(kd.matmul_arrangement, kd.matmul_application, tuple(Tensor(2) for _ in range(3)),
                         caller="cuda", kernel_name="m", output_dir=tmp_path)
    with pytest.raises(aot.AotError):  # is_causal without a value
        t = lambda: Tensor(4, dtype=ninetoothed.float16)  # noqa: E731
        ninetoothed.make(kd.attention_arrangement, kd.attention_application,
                         (t(), t(), t(), Tensor(0, constexpr=True), t()), caller="cuda", kernel_name="a",
                         output_dir=tmp_path)
    with pytest.raises(aot.AotError):  # a name that is not a C identifier
        make_addmm(tmp_path, name="addmm-aot")
    with pytest.raises(ValueError):
        ninetoothed.make(kd.matmul_arrangement, kd.matmul_application, tuple(Tensor(2) for _ in range(3)),
                         caller="cpu")


@pytest.mark.gpu
def test_addmm_through_both_loaders(tmp_path):
    import torch

    from gpu_util import assert_close, assert_device_healthy, dev
    from oracle import inputs as oi
    from oracle import kernels as ok

    ours = make_addmm(tmp_path)
    c, a, b = oi.addmm_inputs(192, 320, 256, 21)
    expected = ok.addmm(c, a, b, 0.5, 2.0)
    out = torch.empty(192, 320, dtype=torch.float16, device="cuda")
    ours(dev(c), dev(a), dev(b), 0.5, 2.0, out)  # Python floats: host doubles
    assert_close(out.cpu().numpy(), expected)
    load = reference_loader()
    if load is not None:
        theirs = load("addmm_aot", tmp_path)
        out.zero_()
        theirs(dev(c), dev(a), dev(b), 0.5, 2.0, out)
        assert_close(out.cpu().numpy(), expected)
    # scalars declared float16 arrive as host fp16 tensors, as in the reference's AOT test
    half = make_addmm(tmp_path, name="addmm_aot_half_scalars", scalar_dtype=ninetoothed.float16)
    out.zero_()
    half(dev(c), dev(a), dev(b), torch.tensor(0.5, dtype=torch.float16), torch.tensor(2.0, dtype=torch.float16), out)
    assert_close(out.cpu().numpy(), expected)
    assert_device_healthy()


@pytest.mark.gpu
def test_matmul_attention_and_conv2d_ahead_of_time(tmp_path):
    import torch

    from gpu_util import assert_close, assert_device_healthy, dev
    from oracle import inputs as oi
    from oracle import kernels as ok

    f16 = ninetoothed.float16
    matmul = ninetoothed.make(kd.matmul_arrangement, kd.matmul_application, tuple(Tensor(2, dtype=f16) for _ in range(3)),
                              caller="cuda", kernel_name="matmul_aot", output_dir=tmp_path)
    a, b = oi.matmul_inputs(256, 128, 192, 22)
    out = torch.empty(256, 128, dtype=torch.float16, device="cuda")
    matmul(dev(a), dev(b), out)
    assert_close(out.cpu().numpy(), ok.matmul(a, b))

    t = lambda: Tensor(4, dtype=f16)  # noqa: E731
    attention = ninetoothed.make(kd.attention_arrangement, kd.attention_application,
                                 (t(), t(), t(), Tensor(0, constexpr=True, value=1), t()), caller="cuda",
                                 kernel_name="attention_aot", output_dir=tmp_path)
    q, k, v = oi.attention_inputs((1, 2, 200, 64), 23)
    o = torch.empty(1, 2, 200, 64, dtype=torch.float16, device="cuda")
    attention(dev(q), dev(k), dev(v), torch.tensor(True), o)  # the flag's value was compiled in
    assert_close(o.cpu().numpy(), ok.attention(q, k, v, True, 64, 64))

    arrangement, application, tensors = kd.conv2d_premake(dtype=f16)
    conv2d = ninetoothed.make(arrangement, application, tensors, caller="cuda", kernel_name="conv2d_aot",
                              output_dir=tmp_path)
    x, w = oi.conv2d_inputs((2, 16, 12, 12), (32, 16, 3, 3), 24)
    y = torch.empty(2, 32, 10, 10, dtype=torch.float16, device="cuda")
    conv2d(dev(x), dev(w), y)
    assert_close(y.cpu().numpy(), ok.conv2d(x, w, (0, 0), block_m=64, block_n=64, block_k=64))
    assert_device_healthy()
