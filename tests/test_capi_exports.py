"""The shared library loads without a GPU and exports every symbol the header declares."""

import ctypes
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "ninetoothed_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    text = "\n".join(line for line in text.splitlines() if not line.lstrip().startswith("#"))
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(names))


@pytest.fixture(scope="module")
def library():
    from ninetoothed_b200 import compile as library_compile

    return ctypes.CDLL(str(library_compile.build()))


def test_header_declares_the_expected_entry_points():
    from ninetoothed_b200 import _capi

    assert set(declared_functions()) == set(_capi.ENTRY_POINTS)


def test_every_declared_symbol_is_exported(library):
    for name in declared_functions():
        assert getattr(library, name) is not None, name


def test_version_and_error_text_without_a_device(library):
    assert library.ninetoothed_b200_version() >= 100
    library.ninetoothed_b200_last_error.restype = ctypes.c_char_p
    assert isinstance(library.ninetoothed_b200_last_error(), bytes)


def test_struct_layout_matches_the_reference_header():
    """{void *data; uint64_t *shape; int64_t *strides;} (src/ninetoothed/aot.py:569-573)."""
    from ninetoothed_b200._capi import NineToothedTensor

    assert [name for name, _ in NineToothedTensor._fields_] == ["data", "shape", "strides"]
    assert ctypes.sizeof(NineToothedTensor) == 3 * ctypes.sizeof(ctypes.c_void_p)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ninetoothed_b200 import _capi

    monkeypatch.setattr(_capi, "_library", None)
    monkeypatch.setattr(_capi, "LIBRARY_PATH", tmp_path / "absent.so")
    with pytest.raises(_capi.LibraryNotBuiltError):
        _capi.library()


def test_cpu_tensors_are_rejected():
    import torch

    from ninetoothed_b200 import _capi

    x = torch.zeros(4, 8, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        _capi.softmax(x, torch.empty_like(x))


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C (a C host includes it directly)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    source = tmp_path / "use.c"
    source.write_text(
        '#include "ninetoothed_b200.h"\n'
        "int use(NineToothedStream s, NineToothedTensor a, NineToothedTensor b, NineToothedTensor c) {\n"
        "    return launch_matmul(s, a, b, c, NINETOOTHED_FLOAT16) + (int)sizeof(NineToothedTensor)\n"
        "           + NINETOOTHED_B200_FLOAT8_E5M2 + (int)NINETOOTHED_B200_STATIC_WORKSPACE_BYTES;\n"
        "}\n")
    include = pathlib.Path(__file__).resolve().parent.parent / "include"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-fsyntax-only", f"-I{include}", str(source)], check=True)


def test_bindings_reject_mixed_dtypes_and_wrong_ranks_before_touching_the_device():
    """The launchers take one dtype tag and index shape[] blindly: a mixed or mis-ranked call must raise
    in the binding (CPU tensors are enough to see it: the checks come before the device is looked at)."""
    import torch

    from ninetoothed_b200 import _capi

    h = lambda *shape: torch.zeros(*shape, dtype=torch.float16)  # noqa: E731
    f = lambda *shape: torch.zeros(*shape, dtype=torch.float32)  # noqa: E731
    b = lambda *shape: torch.zeros(*shape, dtype=torch.bfloat16)  # noqa: E731
    with pytest.raises(TypeError):  # fp16 operands, fp32 output
        _capi.matmul(h(4, 8), h(8, 4), f(4, 4))
    with pytest.raises(TypeError):  # fp16 / bf16 operands
        _capi.matmul(h(4, 8), b(8, 4), h(4, 4))
    with pytest.raises(ValueError):  # a 1-D operand
        _capi.matmul(h(8), h(8, 4), h(4, 4))
    with pytest.raises(TypeError):
        _capi.addmm(f(4, 4), h(4, 8), h(8, 4), 1.0, 1.0, h(4, 4))
    with pytest.raises(ValueError):
        _capi.addmm(h(4), h(4, 8), h(8, 4), 1.0, 1.0, h(4, 4))
    with pytest.raises(TypeError):
        _capi.softmax(h(4, 8), f(4, 8))
    with pytest.raises(ValueError):
        _capi.softmax(h(4, 8, 1), h(4, 8, 1))
    with pytest.raises(TypeError):
        _capi.attention(h(1, 1, 8, 64), h(1, 1, 8, 64), b(1, 1, 8, 64), False, h(1, 1, 8, 64))
    with pytest.raises(ValueError):
        _capi.attention(h(1, 8, 64), h(1, 8, 64), h(1, 8, 64), False, h(1, 8, 64))
    with pytest.raises(TypeError):
        _capi.conv2d(h(1, 8, 6, 6), h(8, 8, 3, 3), f(1, 8, 4, 4), 0, 0)
    with pytest.raises(ValueError):
        _capi.conv2d(h(8, 6, 6), h(8, 8, 3, 3), h(1, 8, 4, 4), 0, 0)
    with pytest.raises(TypeError):
        _capi.max_pool2d(h(1, 1, 4, 4), b(1, 1, 2, 2), 2, 2, False)
    if hasattr(torch, "float8_e5m2"):
        e = lambda *shape: torch.zeros(*shape, dtype=torch.float8_e5m2)  # noqa: E731
        with pytest.raises(TypeError):  # 8-bit operands write fp16 only
            _capi.matmul(e(4, 8), e(8, 4), b(4, 4))
        with pytest.raises(RuntimeError, match="CUDA tensors only"):  # e5m2 -> fp16 passes validation
            _capi.matmul(e(4, 8), e(8, 4), h(4, 4))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):  # a well-formed call gets as far as the device check
        _capi.matmul(h(4, 8), h(8, 4), h(4, 4))


def test_the_multicast_all_gather_refuses_slabs_it_cannot_store_in_whole_steps():
    """The entry point checks the slab's layout before it looks for a device: every store on that path is a whole
    16-byte multimem.st, so ragged or unaligned slabs belong to the peer-store entry point."""
    import torch

    from ninetoothed_b200 import _capi

    def call(width, multicast_address, row_stride=None):
        m, k = 128, 64
        row_stride = width if row_stride is None else row_stride
        slab = torch.zeros(m, row_stride, dtype=torch.float16)[:, :width]
        keep = [_capi.tensor_arg(t) for t in (slab, torch.zeros(m, k, dtype=torch.float16),
                                              torch.zeros(k, width, dtype=torch.float16), slab)]
        beta, alpha = _capi.scalar_arg(1.0), _capi.scalar_arg(1.0)
        return _capi.library().launch_addmm_allgather_multicast(
            None, keep[0][0], keep[1][0], keep[2][0], beta[0], alpha[0], keep[3][0],
            ctypes.c_void_p(multicast_address), 8)

    assert call(64, 0) == -4                       # no multicast address
    assert call(96, 0x1000) == -3                  # not whole 64-column steps
    assert call(64, 0x1008) == -3                  # multicast address not 16-byte aligned
    assert call(64, 0x1000, row_stride=68) == -3   # rows not 16-byte aligned
    assert b"launch_addmm_allgather" in _capi.library().ninetoothed_b200_last_error()


def test_the_mixed_width_planner(monkeypatch):
    """Which launches trade 256-column tiles for 192-column ones, on 74 resident CTA pairs (a B200): the planner is
    host code and needs no device."""
    from ninetoothed_b200 import _capi

    monkeypatch.delenv("NINETOOTHED_B200_GEMM_MIXED", raising=False)
    mib = 1 << 20
    # 8192^3: 1024 tiles are 13.8 waves, nothing to gain
    assert _capi.plan_mixed_widths(32, 32, 74, 4 * mib) == (0, 0, 14 * 560)
    # 4096^3: 256 tiles, four waves of 256 columns -> 148 wide + 144 narrow tiles, two waves of each
    rows, swaps, cycles = _capi.plan_mixed_widths(16, 16, 74, 2 * mib)
    assert (rows * swaps, cycles) == (36, 2 * 560 + 2 * 445)
    assert 16 * 16 - 3 * rows * swaps == 148 and 4 * rows * swaps == 144
    # 8192 x 1024 x 8192: the 18 tile-rows it would take hold 72 MiB of A panels, more than L2 keeps for a second read
    assert _capi.plan_mixed_widths(32, 4, 74, 4 * mib)[:2] == (0, 0)
    assert _capi.plan_mixed_widths(32, 4, 74, 1 * mib)[:2] == (18, 1)      # the same tiles with K = 2048
    # fewer than three column tiles: nothing to swap; fewer tiles than pairs: nothing to fill
    assert _capi.plan_mixed_widths(64, 2, 74, mib)[:2] == (0, 0)
    assert _capi.plan_mixed_widths(4, 4, 74, mib)[:2] == (0, 0)
    monkeypatch.setenv("NINETOOTHED_B200_GEMM_MIXED", "0")
    assert _capi.plan_mixed_widths(16, 16, 74, 2 * mib)[:2] == (0, 0)
    monkeypatch.setenv("NINETOOTHED_B200_GEMM_MIXED", "force")
    assert _capi.plan_mixed_widths(16, 16, 74, 2 * mib)[:2] == (16, 5)
