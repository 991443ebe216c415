"""``make(..., caller="cuda")``: a per-kernel shared library with the reference's AOT shape.

The reference's ahead-of-time path (``src/ninetoothed/aot.py:18-44`` in the reference project)
writes ``<kernel_name>.h`` and ``<kernel_name>.so`` into ``output_dir``; the header declares

    NineToothedResult launch_<kernel_name>(NineToothedStream stream, NineToothedTensor a, ...);

(``aot.py:126-147``) and the reference's own loader (``aot.py:802-862``) reads that line to learn how
many arguments are tensors, opens the library with ctypes and calls the symbol.  This module produces
the same two files for the kernels this library holds: the ``.so`` is a few lines of C++ that forward
to ``launch_<op>`` in ``libninetoothed_b200.so`` (linked by absolute path, found again through an
rpath), with what the reference fixes at compile time fixed here too: the element type (the tensors'
``dtype``) and the value of ``constexpr`` scalars such as ``is_causal``.  A C or C++ host, or the
reference's loader, can use the pair exactly as it would use the reference's output.

Scalars follow the reference's convention (``aot.py:262-281, 838-852``): a 0-dim tensor argument points
at one HOST value of the tensor's declared dtype, float32 being passed as a double and a tensor
without a dtype as a double (floats) or int64 (integers).
"""

from __future__ import annotations

import ctypes
import pathlib
import re
import shutil
import subprocess
import tempfile

from ninetoothed_b200 import compile as library_build
from ninetoothed_b200 import dtype as _dtype

_DTYPE_ENUM = {
    _dtype.int8: "NINETOOTHED_INT8", _dtype.int16: "NINETOOTHED_INT16", _dtype.int32: "NINETOOTHED_INT32",
    _dtype.int64: "NINETOOTHED_INT64", _dtype.uint8: "NINETOOTHED_UINT8", _dtype.uint16: "NINETOOTHED_UINT16",
    _dtype.uint32: "NINETOOTHED_UINT32", _dtype.uint64: "NINETOOTHED_UINT64", _dtype.float16: "NINETOOTHED_FLOAT16",
    _dtype.bfloat16: "NINETOOTHED_BFLOAT16", _dtype.float32: "NINETOOTHED_FLOAT32",
    _dtype.float64: "NINETOOTHED_FLOAT64",
}
_DTYPE_TO_INDEX = {tag: index for index, tag in enumerate(_DTYPE_ENUM)}

# How the forwarder reads one host scalar of each declared dtype into a double.
_SCALAR_READERS = '''
static double nt_half_bits(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31, exponent = (h >> 10) & 31u, mantissa = h & 1023u;
    uint32_t bits;
    if (exponent == 0) {
        if (mantissa == 0) {
            bits = sign;
        } else {  /* subnormal: renormalise */
            int shift = 0;
            uint32_t m = mantissa;
            while (!(m & 1024u)) { m <<= 1; ++shift; }
            bits = sign | ((uint32_t)(113 - shift) << 23) | ((m & 1023u) << 13);
        }
    } else if (exponent == 31) {
        bits = sign | 0x7f800000u | (mantissa << 13);
    } else {
        bits = sign | ((exponent + 112u) << 23) | (mantissa << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}
static double nt_bfloat_bits(uint16_t h) {
    const uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}
'''
_READ_AS_DOUBLE = {
    None: "*(const double *)%s.data",
    _dtype.float64: "*(const double *)%s.data",
    _dtype.float32: "*(const double *)%s.data",  # the reference passes float32 scalars as doubles
    _dtype.float16: "nt_half_bits(*(const uint16_t *)%s.data)",
    _dtype.bfloat16: "nt_bfloat_bits(*(const uint16_t *)%s.data)",
    _dtype.int64: "(double)*(const int64_t *)%s.data",
    _dtype.int32: "(double)*(const int32_t *)%s.data",
}


class AotError(ValueError):
    """The pair is recognised but cannot be fixed ahead of time the way the reference does it."""


def _tensor_dtype(tensors, kernel_name):
    tags = {t.element_type for t in tensors if t.spec_ndim > 0}
    if len(tags) != 1 or None in tags:
        raise AotError(f"{kernel_name}: an ahead-of-time kernel needs one dtype on every tensor "
                       f"(Tensor(ndim, dtype=ninetoothed_b200.float16)), got {sorted(map(str, tags))}")
    tag = tags.pop()
    if tag not in (_dtype.float16, _dtype.bfloat16, _dtype.float32):
        raise AotError(f"{kernel_name}: dtype {tag!r} is not one the kernels compute in")
    return tag


def _forwarder_body(op, names, tensors, dtype_enum, kernel_name):
    """The C++ statements of ``launch_<kernel_name>`` for the recognised ``op``."""

    def scalar(index):
        spec = tensors[index]
        reader = _READ_AS_DOUBLE.get(spec.element_type)
        if reader is None:
            raise AotError(f"{kernel_name}: scalar {names[index]!r} has dtype {spec.element_type!r}")
        return reader % names[index]

    def baked(index, what):
        spec = tensors[index]
        if not spec.constexpr or spec.value is None:
            raise AotError(f"{kernel_name}: {what} {names[index]!r} must be Tensor(0, constexpr=True, value=...) for "
                           "an ahead-of-time kernel: the reference compiles the value in")
        return int(spec.value)

    host_scalar = ("    double {0}_value = {1};\n"
                   "    NineToothedTensor {0}_host = {{&{0}_value, {0}.shape, {0}.strides}};\n")
    if op == "matmul":
        return f"    return launch_matmul(stream, {names[0]}, {names[1]}, {names[2]}, {dtype_enum});\n"
    if op == "bmm":
        return f"    return launch_bmm(stream, {names[0]}, {names[1]}, {names[2]}, {dtype_enum});\n"
    if op == "addmm":
        return (host_scalar.format(names[3], scalar(3)) + host_scalar.format(names[4], scalar(4))
                + f"    return launch_addmm(stream, {names[0]}, {names[1]}, {names[2]}, {names[3]}_host, "
                  f"{names[4]}_host, {names[5]}, {dtype_enum});\n")
    if op == "softmax":
        return f"    return launch_softmax(stream, {names[0]}, {names[1]}, {dtype_enum});\n"
    if op in ("attention", "attention_scaled"):
        causal_at = 4 if op == "attention_scaled" else 3
        text = (f"    int64_t causal_value = {baked(causal_at, 'the causal flag')};\n"
                f"    NineToothedTensor causal_host = {{&causal_value, {names[causal_at]}.shape, "
                f"{names[causal_at]}.strides}};\n")
        if op == "attention":
            return text + (f"    return launch_attention(stream, {names[0]}, {names[1]}, {names[2]}, causal_host, "
                           f"{names[4]}, {dtype_enum});\n")
        return text + host_scalar.format(names[3], scalar(3)) + (
            f"    return launch_attention_scaled(stream, {names[0]}, {names[1]}, {names[2]}, {names[3]}_host, "
            f"causal_host, {names[5]}, {dtype_enum});\n")
    if op == "conv2d":
        return (f"    /* unpadded: the arrangement pads with nothing.  Scratch for the layout pass comes from the\n"
                f"       array built into the library (launch_conv2d_static_workspace). */\n"
                f"    return launch_conv2d_static_workspace(stream, {names[0]}, {names[1]}, {names[2]}, 0, 0, "
                f"{dtype_enum});\n")
    raise AotError(f"{kernel_name}: no ahead-of-time form for {op}")


def generate(recognised, parameters, tensors, kernel_name, output_dir):
    """Write ``<kernel_name>.h``, ``<kernel_name>.cpp`` and ``<kernel_name>.so`` into ``output_dir``."""
    if not kernel_name or not re.fullmatch(r"[A-Za-z_][A-Za-z0-9_]*", kernel_name):
        raise AotError(f"kernel_name {kernel_name!r} must be a C identifier")
    from ninetoothed_b200 import _capi

    if f"launch_{kernel_name}" in _capi.ENTRY_POINTS:
        raise AotError(f"kernel_name {kernel_name!r} is taken: launch_{kernel_name} is an entry point of "
                       "libninetoothed_b200.so itself, which the generated library links against")
    if output_dir is None:
        raise AotError("output_dir is required for a caller other than 'torch'")
    if recognised.constexpr_names:
        raise AotError(f"{kernel_name}: the arrangement leaves {recognised.constexpr_names} to be given per call; an "
                       "ahead-of-time kernel needs them fixed in the arrangement (the reference compiles them in)")
    output_dir = pathlib.Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    names = [re.sub(r"\W", "_", name) for name in parameters]
    dtype_enum = _DTYPE_ENUM[_tensor_dtype(tensors, kernel_name)]
    body = _forwarder_body(recognised.op, names, tensors, dtype_enum, kernel_name)
    library = library_build.build()
    header = library_build.INCLUDE_DIR / "ninetoothed_b200.h"
    params = ", ".join(["NineToothedStream stream"] + [f"NineToothedTensor {name}" for name in names])
    signature = f"NineToothedResult launch_{kernel_name}({params})"
    guard = f"NINETOOTHED_{kernel_name.upper()}_H"
    (output_dir / f"{kernel_name}.h").write_text(
        f"#ifndef {guard}\n#define {guard}\n\n#include \"{header}\"\n\n"
        f"#ifdef __cplusplus\nextern \"C\" {signature};\n#else\n{signature};\n#endif\n\n#endif\n")
    source = output_dir / f"{kernel_name}.cpp"
    source.write_text(
        f"// Forwards launch_{kernel_name} to the {recognised.op} kernel of libninetoothed_b200.so.\n"
        f"#include <stdint.h>\n#include <string.h>\n\n#include \"{header}\"\n{_SCALAR_READERS}\n"
        f"extern \"C\" {signature} {{\n{body}}}\n")
    shared = output_dir / f"{kernel_name}.so"
    compiler = shutil.which("g++") or shutil.which("c++")
    if compiler is None:
        raise AotError("no C++ compiler (g++) on PATH to build the forwarding library")
    command = [compiler, "-shared", "-fPIC", "-O2", str(source), "-o", str(shared), f"-L{library.parent}",
               f"-l:{library.name}", f"-Wl,-rpath,{library.parent}"]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise AotError(f"building {shared} failed:\n{done.stderr}")
    return shared


class KernelLaunchError(RuntimeError):
    """Counterpart of the reference's ``_KernelLaunchError`` (``src/ninetoothed/aot.py:747-751``)."""

    def __init__(self, error_code):
        self.error_code = error_code
        super().__init__(f"Kernel launch failed with error code: {error_code}.")


class _ArgumentTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("shape", ctypes.POINTER(ctypes.c_uint64)),
                ("strides", ctypes.POINTER(ctypes.c_int64))]


def load(kernel_name, output_dir):
    """What the reference's ``_load_launch_func`` does (``aot.py:802-862``): count the tensor parameters
    in ``<kernel_name>.h``, open ``<kernel_name>.so`` (through a temporary copy, so that the file may be
    rebuilt while loaded), and return ``run(*args)`` that marshals torch tensors, Python floats and ints
    (host scalars) and dtype tags, launches on torch's current stream and raises on a non-zero result."""
    import torch

    output_dir = pathlib.Path(output_dir)
    text = (output_dir / f"{kernel_name}.h").read_text()
    match = re.search(rf"NineToothedResult\s+launch_{re.escape(kernel_name)}\s*\((.*?)\)\s*;", text)
    if match is None:
        raise RuntimeError(f"Could not find launch signature for `{kernel_name}` in `{output_dir / (kernel_name + '.h')}`.")
    num_tensor_args = sum(1 for p in match.group(1).split(",") if p.strip().startswith("NineToothedTensor "))
    with tempfile.NamedTemporaryFile(suffix=".so") as copy:
        shutil.copy(output_dir / f"{kernel_name}.so", copy.name)
        library = ctypes.CDLL(copy.name)
    launch = getattr(library, f"launch_{kernel_name}")
    launch.restype = ctypes.c_int
    empty_shape, empty_strides = (ctypes.c_uint64 * 0)(), (ctypes.c_int64 * 0)()

    def marshal(arg, keep):
        if isinstance(arg, torch.Tensor):
            shape = (ctypes.c_uint64 * arg.ndim)(*arg.shape)
            strides = (ctypes.c_int64 * arg.ndim)(*arg.stride())
            keep.append((shape, strides, arg))
            return _ArgumentTensor(arg.data_ptr(), shape, strides)
        if type(arg) in (float, int, bool):
            buffer = ctypes.c_double(arg) if type(arg) is float else ctypes.c_int64(int(arg))
            keep.append(buffer)
            return _ArgumentTensor(ctypes.addressof(buffer), empty_shape, empty_strides)
        return arg

    def run(*args):
        keep, arguments = [], []
        for i, arg in enumerate(args):
            if i < num_tensor_args:
                arguments.append(marshal(arg, keep))
            elif type(arg) is str:
                arguments.append(_DTYPE_TO_INDEX[arg])
            else:
                arguments.append(arg)
        stream = ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))
        result = launch(stream, *arguments)
        if result != 0:
            raise KernelLaunchError(result)

    return run
