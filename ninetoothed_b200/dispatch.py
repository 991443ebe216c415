"""``build``: one callable over several configurations of a kernel.

Mirrors ``ninetoothed.build`` (``src/ninetoothed/build.py:26-215`` in the reference
project).  There, ``premake(*args, **kwargs)`` returns an (arrangement, application,
tensors) triple per configuration, every configuration is compiled ahead of time,
and a generated C dispatcher picks the variant whose parameters equal the trailing
integer arguments of the call (``build.py:147-176, 763-764``); with
``meta_parameters`` an auto-tuner picks those for the caller and keeps a CSV cache
(``build.py:178-215``, ``templates/auto_tuning_cache.h``).

Here every configuration is recognised through ``make`` and bound to the same
hand-scheduled kernel: block sizes, ``num_warps`` and ``num_stages`` do not select
code, the tile shapes are chosen per problem by the tables in the C++ launchers
(``csrc/gemm.cu`` ``launch_shape``, ``csrc/conv2d.cu`` ``run_typed``).  What is kept
is the calling convention and the dispatch rule, so that callers written for the
reference's ``build`` run unchanged:

    kernel = build(premake, configs, caller="cuda", kernel_name="conv2d", output_dir=...)
    kernel(input, filter, output, *config_values)

``config_values`` are the values of premake's bound arguments (defaults applied)
followed by the compilation configuration's, converted to integers the way the
reference does (``build.py:799-812``); a call whose values match no configuration
raises ``KernelLaunchError`` with the reference dispatcher's result code 1.
"""

from __future__ import annotations

import enum
import inspect

from ninetoothed_b200 import dtype as _dtype
from ninetoothed_b200.make import make

# enum NineToothedDataType, by the tags of ninetoothed_b200.dtype (src/ninetoothed/aot.py:524-537)
_DTYPE_TO_INDEX = {
    tag: index
    for index, tag in enumerate((
        _dtype.int8, _dtype.int16, _dtype.int32, _dtype.int64, _dtype.uint8, _dtype.uint16, _dtype.uint32, _dtype.uint64,
        _dtype.float16, _dtype.bfloat16, _dtype.float32, _dtype.float64,
    ))
}


class KernelLaunchError(RuntimeError):
    """Counterpart of the reference's ``_KernelLaunchError`` for a call no configuration matches."""

    def __init__(self, kernel_name, error_code, detail=""):
        self.error_code = error_code
        super().__init__(f"launch_{kernel_name} failed with error code: {error_code}. {detail}".strip())


def _arg_to_int(arg):
    """``build.py:799-812``: ints stay, True/False/None become 1/0/0, dtype tags their enum index,
    enums their value; anything else is compared as it is."""
    if type(arg) is int:
        return arg
    if isinstance(arg, bool) or arg is None:
        return 1 if arg is True else 0
    if isinstance(arg, str) and arg in _DTYPE_TO_INDEX:
        return _DTYPE_TO_INDEX[arg]
    if isinstance(arg, enum.Enum):
        return arg.value
    return arg


class _Variant:
    def __init__(self, handle, combination, num_tensor_params):
        self.handle = handle
        self.combination = combination  # parameter name -> integer value, in dispatch order
        self.num_tensor_params = num_tensor_params


class _BuiltKernel:
    """``kernel(*tensors, *config_values)``: the variant whose parameters equal the trailing values
    is launched on torch's current stream; returns None."""

    def __init__(self, kernel_name, variants, meta_parameters):
        self.kernel_name = kernel_name
        self.variants = tuple(variants)
        self.meta_parameters = tuple(f"{name}" for name in (meta_parameters or ()))
        # The dispatcher's parameter list is the union over the variants, longest signature first
        # (build.py:125-137).
        names = {}
        for variant in sorted(self.variants, key=lambda v: len(v.combination), reverse=True):
            names.update(dict.fromkeys(variant.combination))
        self.param_names = tuple(names)
        self.num_tensor_params = max(v.num_tensor_params for v in self.variants)

    def _is_meta(self, name):
        return name in self.meta_parameters or name.rstrip("_") in self.meta_parameters

    def __call__(self, *args):
        n = self.num_tensor_params
        tensors, trailing = args[:n], tuple(_arg_to_int(a) for a in args[n:])
        names = tuple(name for name in self.param_names if not self._is_meta(name))
        if len(trailing) != len(names):
            raise TypeError(f"launch_{self.kernel_name}() takes {n} tensors and {len(names)} configuration values "
                            f"{names}, got {len(args)} arguments")
        given = dict(zip(names, trailing))
        for variant in self.variants:
            wanted = {k: v for k, v in variant.combination.items() if not self._is_meta(k)}
            if all(given.get(k) == v for k, v in wanted.items()):
                variant.handle(*tensors[:variant.num_tensor_params])
                return None
        raise KernelLaunchError(self.kernel_name, 1, f"no configuration matches {given}")


class _LazyKernel:
    """Defers the build to the first call (``build.py:229-241``)."""

    def __init__(self, factory):
        self._factory, self._kernel = factory, None

    def __call__(self, *args, **kwargs):
        if self._kernel is None:
            self._kernel = self._factory()
        return self._kernel(*args, **kwargs)


def build(premake, configs, *, meta_parameters=None, caller=None, kernel_name=None, output_dir=None, lazy=False):
    """Build a kernel from a ``premake`` function and ``configs``.

    :param premake: Returns ``(arrangement, application, tensors)`` for a configuration.
    :param configs: Iterable of ``(args, kwargs, compilation_configs)``; ``args`` and ``kwargs`` go to
        ``premake``, ``compilation_configs`` to ``make`` (accepted and ignored there).
    :param meta_parameters: Names of premake parameters (or compilation settings) that the caller does
        not pass: the reference auto-tunes them, here they select nothing.
    :param caller: Accepted for signature compatibility (the kernels run on torch CUDA tensors).
    :param kernel_name: Name used in error messages (defaults to the application's).
    :param output_dir: Accepted for signature compatibility; nothing is written.
    :param lazy: Defer the recognition to the first call.
    """
    configs = tuple(configs)
    if not configs:
        raise ValueError("build() needs at least one configuration")
    if lazy:
        return _LazyKernel(lambda: build(premake, configs, meta_parameters=meta_parameters, caller=caller,
                                         kernel_name=kernel_name, output_dir=output_dir))
    signature = inspect.signature(premake)
    variants = []
    for args, kwargs, compilation_configs in configs:
        arrangement, application, tensors = premake(*args, **kwargs)
        bound = signature.bind(*args, **kwargs)
        bound.apply_defaults()
        combination = {f"{name}_": _arg_to_int(value) for name, value in bound.arguments.items()}
        combination.update({name: _arg_to_int(value) for name, value in compilation_configs.items()})
        handle = make(arrangement, application, tensors, kernel_name=kernel_name, **{
            key: value for key, value in compilation_configs.items()
            if key in ("num_warps", "num_stages", "max_num_configs")
        })
        variants.append(_Variant(handle, combination, len(inspect.signature(application).parameters)))
    name = kernel_name or variants[0].handle.kernel_name
    return _BuiltKernel(name, variants, meta_parameters)
