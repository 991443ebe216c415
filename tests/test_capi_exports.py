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
