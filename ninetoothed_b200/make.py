"""``make`` and ``jit``: the front door with the reference's signatures.

``make(arrangement, application, tensors)`` returns a callable that takes the same
torch tensors, scalars and constexpr keywords as the callable the reference
returns (``src/ninetoothed/make.py:7-56``, ``src/ninetoothed/jit.py:8-58, 121-128``
in the reference project), writes the output tensor in place and returns None.
Behind it sits a hand-written sm_100a kernel, reached through a PyTorch custom op
and the C ABI, instead of generated Triton source.  Pairs that are not one of the
kernels this library holds raise ``UnsupportedKernelError``; nothing falls back.
"""

from __future__ import annotations

import inspect

from ninetoothed_b200.recognition import Recognised, UnsupportedKernelError, recognise, recognise_application, \
    recognise_arrangement
from ninetoothed_b200.tensor import Tensor


class _Handle:
    """What ``make``/``jit`` return.  ``handle(*tensors, **constexprs)`` launches on
    torch's current stream and returns None (``src/ninetoothed/jit.py:121-128``)."""

    def __init__(self, recognised: Recognised, parameters, kernel_name):
        self.op = recognised.op
        self.block_sizes = dict(recognised.block_sizes)
        self.constexpr_names = tuple(recognised.constexpr_names)
        self.parameters = tuple(parameters)
        self.kernel_name = kernel_name
        self._padded = recognised.padded
        self._ceil_mode = recognised.ceil_mode

    def __repr__(self):
        return f"<ninetoothed_b200 kernel {self.kernel_name!r}: {self.op}>"

    def _bind(self, args, kwargs):
        n = len(self.parameters)
        if len(args) < n:
            raise TypeError(f"{self.kernel_name}() takes {n} positional arguments {self.parameters}, got {len(args)}")
        positional, extra = args[:n], args[n:]
        if len(extra) > len(self.constexpr_names):
            raise TypeError(f"{self.kernel_name}() got {len(args)} positional arguments, at most "
                            f"{n + len(self.constexpr_names)} expected")
        constexprs = dict(zip(self.constexpr_names, extra))
        for name, value in kwargs.items():
            if name not in self.constexpr_names:
                raise TypeError(f"{self.kernel_name}() got an unexpected keyword argument {name!r}")
            if name in constexprs:
                raise TypeError(f"{self.kernel_name}() got multiple values for argument {name!r}")
            constexprs[name] = value
        missing = [name for name in self.constexpr_names if name not in constexprs]
        if missing:
            raise TypeError(f"{self.kernel_name}() missing constexpr argument(s) {missing}")
        return positional, constexprs

    def __call__(self, *args, **kwargs):
        from ninetoothed_b200.torch_ops import ops

        a, constexprs = self._bind(args, kwargs)
        if self.op == "matmul":
            ops.matmul(a[0], a[1], a[2])
        elif self.op == "bmm":
            ops.bmm(a[0], a[1], a[2])
        elif self.op == "addmm":
            ops.addmm(a[0], a[1], a[2], float(a[3]), float(a[4]), a[5])
        elif self.op == "softmax":
            block = int(constexprs["BLOCK_SIZE"]) if "BLOCK_SIZE" in constexprs else self.block_sizes["BLOCK_SIZE"]
            if "BLOCK_SIZE" in constexprs and block < a[0].shape[-1]:
                raise UnsupportedKernelError(
                    f"softmax: BLOCK_SIZE={block} is smaller than the row length {a[0].shape[-1]}; the kernel "
                    "normalises whole rows (one program per row)"
                )
            ops.softmax(a[0], a[1])
        elif self.op == "attention":
            ops.attention(a[0], a[1], a[2], bool(a[3]), a[4])
        elif self.op == "attention_scaled":
            ops.attention_scaled(a[0], a[1], a[2], float(a[3]), bool(a[4]), a[5])
        elif self.op == "conv2d":
            ops.conv2d(a[0], a[1], a[2], int(constexprs.get("padding_h", 0)), int(constexprs.get("padding_w", 0)))
        elif self.op == "max_pool2d":
            ops.max_pool2d(a[0], a[1], int(constexprs["WINDOW_HEIGHT"]), int(constexprs["WINDOW_WIDTH"]), self._ceil_mode)
        else:  # pragma: no cover
            raise AssertionError(self.op)
        return None


def make(arrangement, application, tensors, caller="torch", kernel_name=None, output_dir=None, num_warps=None,
         num_stages=None, max_num_configs=None):
    """Integrate the arrangement and the application of the tensors.

    :param arrangement: The arrangement of the tensors.
    :param application: The application of the tensors.
    :param tensors: The tensors.
    :param caller: Who will call the compute kernel: ``"torch"`` (a handle for torch tensors) or
        ``"cuda"`` (ahead of time: ``<kernel_name>.h`` and ``<kernel_name>.so`` are written to
        ``output_dir`` in the reference's AOT shape, and a loader for them is returned).
    :param kernel_name: The name for the kernel (defaults to the application's).
    :param output_dir: Where the ahead-of-time files go (``caller="cuda"`` only).
    :param num_warps: Accepted and ignored: the kernels are hand-scheduled.
    :param num_stages: Accepted and ignored.
    :param max_num_configs: Accepted and ignored: there is no auto-tuning.
    :return: A handle to the compute kernel.
    """
    if caller not in ("torch", "cuda"):
        raise ValueError(f"unsupported caller {caller!r}: this library runs on CUDA devices only "
                         "('torch' for a torch handle, 'cuda' for an ahead-of-time library)")
    tensors = tuple(tensors)
    recognised = recognise(arrangement, application, tensors)
    parameters = tuple(inspect.signature(application).parameters)
    if len(parameters) != len(tensors):
        raise ValueError(f"the application takes {len(parameters)} parameters but {len(tensors)} tensors were given")
    kernel_name = kernel_name or application.__name__
    if caller == "cuda":
        # src/ninetoothed/make.py:48-56 and aot.py:18-44 in the reference project: write the files, load them back
        from ninetoothed_b200 import aot

        aot.generate(recognised, parameters, tensors, kernel_name, output_dir)
        return aot.load(kernel_name, output_dir)
    return _Handle(recognised, parameters, kernel_name)


def jit(func=None, *, caller="torch", kernel_name=None, num_warps=None, num_stages=None, max_num_configs=None,
        _prettify=False):
    """Decorator form: the parameter annotations of ``func`` are the arranged tensors
    (``src/ninetoothed/jit.py:8-58``; used by ``tests/test_softmax.py:13-21``)."""

    def wrapper(func):
        if caller != "torch":
            raise ValueError(f"unsupported caller {caller!r}")
        annotations = inspect.get_annotations(func)
        parameters = tuple(inspect.signature(func).parameters)
        specs = []
        for name in parameters:
            spec = annotations.get(name)
            if not isinstance(spec, Tensor):
                raise TypeError(f"parameter {name!r} of {func.__name__} must be annotated with an arranged Tensor")
            specs.append(spec)

        def arrangement(*bound):
            # `instantiate` already replayed the meta-operations recorded on each annotation
            return tuple(bound)

        arranged = recognise_arrangement(arrangement, specs)
        applied = recognise_application(func)
        if arranged.op != applied:
            raise UnsupportedKernelError(f"the annotations tile like {arranged.op} but the body computes {applied}")
        return _Handle(arranged, parameters, kernel_name or func.__name__)

    if func is None:
        return wrapper
    return wrapper(func)
