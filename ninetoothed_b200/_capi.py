"""ctypes binding of ``libninetoothed_b200.so`` (the C ABI in ``include/ninetoothed_b200.h``).

Marshals torch tensors into ``NineToothedTensor`` structs the way the reference's
AOT loader does (``src/ninetoothed/aot.py:711-733, 838-862`` in the reference
project): tensors become ``{data_ptr, shape[], strides[]}``, Python floats become
0-dim tensors pointing at a host ``double``, ints/bools at a host ``int64``; the
stream is torch's current raw stream; a non-zero result raises.

There is no fallback: if the library is missing or a call fails, this raises.
"""

from __future__ import annotations

import ctypes
import pathlib
import threading
import warnings

import torch

LIBRARY_PATH = pathlib.Path(__file__).resolve().parent / "lib" / "libninetoothed_b200.so"

# enum NineToothedDataType (same order as the reference, src/ninetoothed/aot.py:524-537)
DTYPE_INDEX = {
    torch.int8: 0, torch.int16: 1, torch.int32: 2, torch.int64: 3,
    torch.uint8: 4, torch.uint16: 5, torch.uint32: 6, torch.uint64: 7,
    torch.float16: 8, torch.bfloat16: 9, torch.float32: 10, torch.float64: 11,
}
if hasattr(torch, "float8_e5m2"):
    DTYPE_INDEX[torch.float8_e5m2] = 100  # NINETOOTHED_B200_FLOAT8_E5M2 (not in the reference's enum)

ENTRY_POINTS = (
    "launch_matmul",
    "launch_bmm",
    "launch_addmm",
    "launch_addmm_allgather",
    "launch_addmm_allgather_multicast",
    "launch_softmax",
    "launch_attention",
    "launch_attention_scaled",
    "launch_conv2d",
    "launch_conv2d_workspace_size",
    "launch_conv2d_static_workspace",
    "launch_max_pool2d",
    "ninetoothed_b200_last_error",
    "ninetoothed_b200_device_status",
    "ninetoothed_b200_selftest_wait_timeout",
    "ninetoothed_b200_reserve_split_scratch",
    "ninetoothed_b200_plain_launches",
    "ninetoothed_b200_mixed_width_launches",
    "ninetoothed_b200_plan_mixed_widths",
    "ninetoothed_b200_last_note",
    "ninetoothed_b200_version",
)

ERR_TIMEOUT = -6  # NINETOOTHED_B200_ERR_TIMEOUT


class SlowPathWarning(UserWarning):
    """A launch ran on a plain CUDA-core kernel instead of the tensor-core path."""


class NineToothedTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("shape", ctypes.POINTER(ctypes.c_uint64)),
        ("strides", ctypes.POINTER(ctypes.c_int64)),
    ]


class KernelLaunchError(RuntimeError):
    """Counterpart of the reference's ``_KernelLaunchError`` (``src/ninetoothed/aot.py:747-751``)."""

    def __init__(self, entry_point, error_code, detail):
        self.error_code = error_code
        super().__init__(f"{entry_point} failed with error code: {error_code}. {detail}".strip())


class LibraryNotBuiltError(RuntimeError):
    pass


_EMPTY_SHAPE = (ctypes.c_uint64 * 0)()
_EMPTY_STRIDES = (ctypes.c_int64 * 0)()

_lock = threading.Lock()
_library = None


def library() -> ctypes.CDLL:
    """The loaded shared library; raises when it has not been built."""
    global _library
    if _library is not None:
        return _library
    with _lock:
        if _library is None:
            if not LIBRARY_PATH.exists():
                raise LibraryNotBuiltError(
                    f"{LIBRARY_PATH} does not exist: build it with `python -m ninetoothed_b200.compile` "
                    "(there is no CPU or library fallback)"
                )
            lib = ctypes.CDLL(str(LIBRARY_PATH))
            T, S, I = NineToothedTensor, ctypes.c_void_p, ctypes.c_int
            lib.launch_matmul.argtypes = [S, T, T, T, I]
            lib.launch_bmm.argtypes = [S, T, T, T, I]
            lib.launch_addmm.argtypes = [S, T, T, T, T, T, T, I]
            lib.launch_addmm_allgather.argtypes = [S, T, T, T, T, T, T, ctypes.POINTER(ctypes.c_void_p), I, I, I]
            lib.launch_addmm_allgather_multicast.argtypes = [S, T, T, T, T, T, T, ctypes.c_void_p, I]
            lib.launch_softmax.argtypes = [S, T, T, I]
            lib.launch_attention.argtypes = [S, T, T, T, T, T, I]
            lib.launch_attention_scaled.argtypes = [S, T, T, T, T, T, T, I]
            lib.launch_conv2d.argtypes = [S, T, T, T, I, I, I, ctypes.c_void_p, ctypes.c_size_t]
            lib.launch_conv2d_workspace_size.argtypes = [T, T, I]
            lib.launch_conv2d_static_workspace.argtypes = [S, T, T, T, I, I, I]
            lib.launch_max_pool2d.argtypes = [S, T, T, I, I, I, I]
            lib.launch_conv2d_workspace_size.restype = ctypes.c_size_t
            lib.ninetoothed_b200_last_error.restype = ctypes.c_char_p
            lib.ninetoothed_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint), I]
            lib.ninetoothed_b200_selftest_wait_timeout.argtypes = [S, ctypes.c_ulonglong]
            lib.ninetoothed_b200_reserve_split_scratch.argtypes = [S]
            lib.ninetoothed_b200_plain_launches.argtypes = [I]
            lib.ninetoothed_b200_plain_launches.restype = ctypes.c_longlong
            lib.ninetoothed_b200_mixed_width_launches.argtypes = [I]
            lib.ninetoothed_b200_mixed_width_launches.restype = ctypes.c_longlong
            lib.ninetoothed_b200_plan_mixed_widths.argtypes = [
                ctypes.c_longlong, ctypes.c_longlong, I, ctypes.c_longlong, ctypes.POINTER(I), ctypes.POINTER(I)]
            lib.ninetoothed_b200_plan_mixed_widths.restype = ctypes.c_longlong
            lib.ninetoothed_b200_last_note.restype = ctypes.c_char_p
            for name in ENTRY_POINTS:
                getattr(lib, name)  # AttributeError here means header and library disagree
            _library = lib
    return _library


_SHAPE_ARRAY = tuple(ctypes.c_uint64 * n for n in range(9))   # array types by rank, made once
_STRIDE_ARRAY = tuple(ctypes.c_int64 * n for n in range(9))


def tensor_arg(t: torch.Tensor):
    """torch tensor -> (struct, keep-alive tuple)."""
    shape = _SHAPE_ARRAY[t.ndim](*t.shape)
    strides = _STRIDE_ARRAY[t.ndim](*t.stride())
    return NineToothedTensor(t.data_ptr(), shape, strides), (shape, strides, t)


def scalar_arg(value):
    """Python / 0-dim torch scalar -> 0-dim NineToothedTensor over a host buffer."""
    if isinstance(value, torch.Tensor):
        value = value.item()
    if isinstance(value, (bool, int)):
        buffer = ctypes.c_int64(int(value))
    else:
        buffer = ctypes.c_double(float(value))
    return NineToothedTensor(ctypes.addressof(buffer), _EMPTY_SHAPE, _EMPTY_STRIDES), (buffer,)


def current_stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device.index))


def check(entry_point: str, result: int):
    if result != 0:
        detail = library().ninetoothed_b200_last_error().decode("utf-8", "replace")
        raise KernelLaunchError(entry_point, result, detail)


def dtype_index(t: torch.Tensor) -> int:
    try:
        return DTYPE_INDEX[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _require_cuda(*tensors):
    device = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("ninetoothed_b200 kernels run on CUDA tensors only (there is no CPU path)")
        if t.device != device:
            raise RuntimeError(f"tensors live on different devices: {device} and {t.device}")
    return device


def _validate(kernel, **tensors):
    """Every tensor of a call has the rank the C side indexes (it reads ``shape[i]`` and
    ``strides[i]`` without a length) and one common dtype (the launchers take a single
    dtype tag and treat every buffer as that type).  Passed as ``label=(tensor, ndim)``;
    checked before anything touches the device, so a bad call raises and corrupts nothing.
    The one mixed case the kernels implement is the 8-bit matmul: e5m2 operands, fp16 output."""
    items = list(tensors.items())
    for label, (t, ndim) in items:
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{kernel}: {label} must be a torch.Tensor, got {type(t).__name__}")
        if t.ndim != ndim:
            raise ValueError(f"{kernel}: {label} must have {ndim} dimensions, got shape {tuple(t.shape)}")
    first_label, (first, _) = items[0]
    e5m2 = getattr(torch, "float8_e5m2", None)
    for label, (t, _) in items[1:]:
        if t.dtype == first.dtype:
            continue
        if kernel == "matmul" and label == "output" and first.dtype == e5m2 and t.dtype == torch.float16 \
                and all(x.dtype == e5m2 for _, (x, _) in items[:-1]):
            continue
        raise TypeError(f"{kernel}: {label} is {t.dtype} but {first_label} is {first.dtype}; every tensor of a call "
                        "must have the same dtype (only the e5m2 matmul writes a different one, float16)")


_plain_launches_seen = 0


def _call(name, device, *args):
    global _plain_launches_seen
    lib = library()
    if torch.cuda.current_device() == device.index:  # (switching the device and back costs more than a small launch)
        check(name, getattr(lib, name)(current_stream(device), *args))
    else:
        with torch.cuda.device(device):
            check(name, getattr(lib, name)(current_stream(device), *args))
    count = lib.ninetoothed_b200_plain_launches(0)
    if count != _plain_launches_seen:  # this launch left the tensor-core path: say so (Python shows it once per site)
        _plain_launches_seen = count
        warnings.warn(lib.ninetoothed_b200_last_note().decode("utf-8", "replace"), SlowPathWarning, stacklevel=3)


def matmul(lhs, rhs, output):
    _validate("matmul", lhs=(lhs, 2), rhs=(rhs, 2), output=(output, 2))
    device = _require_cuda(lhs, rhs, output)
    a, ka = tensor_arg(lhs)
    b, kb = tensor_arg(rhs)
    c, kc = tensor_arg(output)
    _call("launch_matmul", device, a, b, c, dtype_index(lhs))


def bmm(lhs, rhs, output):
    _validate("bmm", lhs=(lhs, 3), rhs=(rhs, 3), output=(output, 3))
    device = _require_cuda(lhs, rhs, output)
    a, ka = tensor_arg(lhs)
    b, kb = tensor_arg(rhs)
    c, kc = tensor_arg(output)
    _call("launch_bmm", device, a, b, c, dtype_index(lhs))


def addmm(input, mat1, mat2, beta, alpha, output):
    _validate("addmm", mat1=(mat1, 2), mat2=(mat2, 2), input=(input, 2), output=(output, 2))
    device = _require_cuda(input, mat1, mat2, output)
    i, ki = tensor_arg(input)
    a, ka = tensor_arg(mat1)
    b, kb = tensor_arg(mat2)
    be, kbe = scalar_arg(float(beta))
    al, kal = scalar_arg(float(alpha))
    c, kc = tensor_arg(output)
    _call("launch_addmm", device, i, a, b, be, al, c, dtype_index(mat1))


def addmm_allgather(input, mat1, mat2, beta, alpha, output_slab, peer_buffer_ptrs, rank):
    """addmm of one rank's column slab with the all-gather fused into the epilogue.

    ``output_slab`` is this rank's [M, N_local] view of its own full buffer;
    ``peer_buffer_ptrs[i]`` is the device address of rank i's full buffer as mapped
    into this process (``peer_buffer_ptrs[rank]`` is this rank's own)."""
    _validate("addmm_allgather", mat1=(mat1, 2), mat2=(mat2, 2), input=(input, 2), output_slab=(output_slab, 2))
    device = _require_cuda(input, mat1, mat2, output_slab)
    i, ki = tensor_arg(input)
    a, ka = tensor_arg(mat1)
    b, kb = tensor_arg(mat2)
    be, kbe = scalar_arg(float(beta))
    al, kal = scalar_arg(float(alpha))
    c, kc = tensor_arg(output_slab)
    world = len(peer_buffer_ptrs)
    ptrs = (ctypes.c_void_p * world)(*peer_buffer_ptrs)
    _call("launch_addmm_allgather", device, i, a, b, be, al, c, ptrs, world, int(rank), dtype_index(mat1))


def addmm_allgather_multicast(input, mat1, mat2, beta, alpha, output_slab, multicast_slab_ptr):
    """The same step with one ``multimem.st`` per 16 bytes: ``multicast_slab_ptr`` is the address of the slab's first
    element in the multicast mapping of the ranks' buffers, and the NVSwitch makes the copies."""
    _validate("addmm_allgather_multicast", mat1=(mat1, 2), mat2=(mat2, 2), input=(input, 2), output_slab=(output_slab, 2))
    device = _require_cuda(input, mat1, mat2, output_slab)
    i, ki = tensor_arg(input)
    a, ka = tensor_arg(mat1)
    b, kb = tensor_arg(mat2)
    be, kbe = scalar_arg(float(beta))
    al, kal = scalar_arg(float(alpha))
    c, kc = tensor_arg(output_slab)
    _call("launch_addmm_allgather_multicast", device, i, a, b, be, al, c, ctypes.c_void_p(int(multicast_slab_ptr)),
          dtype_index(mat1))


def softmax(input, output):
    _validate("softmax", input=(input, 2), output=(output, 2))
    device = _require_cuda(input, output)
    x, kx = tensor_arg(input)
    y, ky = tensor_arg(output)
    _call("launch_softmax", device, x, y, dtype_index(input))


def attention(q, k, v, is_causal, o, scale=None):
    _validate("attention", q=(q, 4), k=(k, 4), v=(v, 4), o=(o, 4))
    device = _require_cuda(q, k, v, o)
    qa, kq = tensor_arg(q)
    ka_, kk = tensor_arg(k)
    va, kv = tensor_arg(v)
    ca, kc = scalar_arg(bool(is_causal))
    oa, ko = tensor_arg(o)
    if scale is None:
        _call("launch_attention", device, qa, ka_, va, ca, oa, dtype_index(q))
    else:
        sa, ks = scalar_arg(float(scale))
        _call("launch_attention_scaled", device, qa, ka_, va, sa, ca, oa, dtype_index(q))


def conv2d_workspace_size(input, filter) -> int:
    _validate("conv2d", input=(input, 4), filter=(filter, 4))
    x, kx = tensor_arg(input)
    w, kw = tensor_arg(filter)
    return int(library().launch_conv2d_workspace_size(x, w, dtype_index(input)))


def conv2d(input, filter, output, padding_h, padding_w, workspace=None):
    _validate("conv2d", input=(input, 4), filter=(filter, 4), output=(output, 4))
    device = _require_cuda(input, filter, output)
    x, kx = tensor_arg(input)
    w, kw = tensor_arg(filter)
    y, ky = tensor_arg(output)
    size = conv2d_workspace_size(input, filter)
    if workspace is None:
        workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=device)
    elif workspace.numel() * workspace.element_size() < size:
        raise ValueError(f"conv2d workspace holds {workspace.numel() * workspace.element_size()} bytes, needs {size}")
    _call("launch_conv2d", device, x, w, y, int(padding_h), int(padding_w), dtype_index(input),
          ctypes.c_void_p(workspace.data_ptr()), ctypes.c_size_t(size))


STATIC_WORKSPACE_BYTES = 32 * 1024 * 1024  # NINETOOTHED_B200_STATIC_WORKSPACE_BYTES


def conv2d_static_workspace(input, filter, output, padding_h, padding_w):
    """conv2d on the scratch array built into the library, for callers that cannot
    allocate device memory (see ``launch_conv2d_static_workspace`` in the header).

    Nothing is allocated here either: the arguments are wrapped in ctypes structs and
    passed through.  Problems whose scratch need exceeds ``STATIC_WORKSPACE_BYTES``
    raise ``KernelLaunchError``; calls on one device share the array, so keep them on
    one stream.  Make the first call on a device outside any stream capture."""
    _validate("conv2d", input=(input, 4), filter=(filter, 4), output=(output, 4))
    device = _require_cuda(input, filter, output)
    x, kx = tensor_arg(input)
    w, kw = tensor_arg(filter)
    y, ky = tensor_arg(output)
    _call("launch_conv2d_static_workspace", device, x, w, y, int(padding_h), int(padding_w), dtype_index(input))


def max_pool2d(input, output, window_height, window_width, ceil_mode):
    _validate("max_pool2d", input=(input, 4), output=(output, 4))
    device = _require_cuda(input, output)
    x, kx = tensor_arg(input)
    y, ky = tensor_arg(output)
    _call("launch_max_pool2d", device, x, y, int(window_height), int(window_width), int(bool(ceil_mode)),
          dtype_index(input))


def device_status(clear=True) -> int:
    """Status word of the current device (0 = no bounded wait ever gave up). Synchronises."""
    status = ctypes.c_uint(0)
    result = library().ninetoothed_b200_device_status(ctypes.byref(status), int(clear))
    if result != ERR_TIMEOUT:  # a give-up code is what this function is asked for: return it, do not raise
        check("ninetoothed_b200_device_status", result)
    return status.value


def device_status_result(clear=True):
    """(result code, status word) exactly as the C entry point returns them."""
    status = ctypes.c_uint(0)
    return library().ninetoothed_b200_device_status(ctypes.byref(status), int(clear)), status.value


def selftest_wait_timeout(limit_ns=5000, device=None):
    """Launch the library's self-test kernel: a bounded wait that runs out after ``limit_ns``."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(device):
        check("ninetoothed_b200_selftest_wait_timeout",
              library().ninetoothed_b200_selftest_wait_timeout(current_stream(device), int(limit_ns)))


def reserve_split_scratch(device=None):
    """Allocate the current stream's scratch for split reductions now, so that no launch allocates later."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(device):
        check("ninetoothed_b200_reserve_split_scratch",
              library().ninetoothed_b200_reserve_split_scratch(current_stream(device)))


def plan_mixed_widths(tile_rows, tile_cols, pairs, row_panel_bytes):
    """(tile-rows that swap, swaps in each, modelled cycles per K-block step of the longest pair); no device needed."""
    rows, swaps = ctypes.c_int(0), ctypes.c_int(0)
    cycles = library().ninetoothed_b200_plan_mixed_widths(tile_rows, tile_cols, pairs, row_panel_bytes,
                                                         ctypes.byref(rows), ctypes.byref(swaps))
    return rows.value, swaps.value, int(cycles)


def mixed_width_launches(reset=False) -> int:
    """Launches that traded 256-column tiles for 192-column ones to fill their last wave."""
    return int(library().ninetoothed_b200_mixed_width_launches(int(reset)))


def plain_launches(reset=False) -> int:
    return int(library().ninetoothed_b200_plain_launches(int(reset)))
