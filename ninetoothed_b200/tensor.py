"""Symbolic tensors and their meta-operations, evaluated on concrete probe shapes.

The constructor and the meta-operations (``tile``, ``expand``, ``squeeze``,
``unsqueeze``, ``permute``, ``flatten``, ``ravel``, ``pad``, ``.dtype``,
``.shape``) have the reference's signatures and meaning
(``src/ninetoothed/tensor.py:11-125, 199-569`` in the reference project), so the
reference's arrangement functions run unchanged.  Instead of building offset
expressions for a code generator, a tensor here carries the *index map* of its
arrangement for one concrete shape: an integer array with one axis per dimension
of every level, holding the flat index of the source element each position reads,
or -1 where the reference's bounds mask is false (partial tiles, padding).  This is
the same object ``Tensor.eval`` yields in the reference (``src/ninetoothed/eval.py:15-58``);
the front door compares it with the index map of the kernels it owns.
"""

from __future__ import annotations

import math

import numpy as np

from ninetoothed_b200.symbol import Symbol

_probe_env: dict | None = None  # symbol name -> value while an arrangement is being probed
_used_symbols: list | None = None


class ProbeScope:
    """Values for symbols while an arrangement runs on probe tensors."""

    def __init__(self, env=None):
        self.env = dict(env or {})
        self.used = []
        self._next_value = 2

    def __enter__(self):
        global _probe_env, _used_symbols
        self._saved = (_probe_env, _used_symbols)
        _probe_env, _used_symbols = self, self.used
        return self

    def __exit__(self, *exc):
        global _probe_env, _used_symbols
        _probe_env, _used_symbols = self._saved

    def value_of(self, symbol: Symbol):
        for name_symbol in symbol.names():
            if name_symbol.name not in self.env:
                # Distinct small values so that distinct block sizes stay distinguishable.
                self.env[name_symbol.name] = self._next_value
                self._next_value += 1
            if name_symbol not in self.used:
                self.used.append(name_symbol)
        return symbol.evaluate(self.env)


def _resolve(value):
    """int for an int or for a symbol under the active probe scope."""
    if isinstance(value, Symbol):
        if _probe_env is None:
            raise RuntimeError("symbols can only be resolved while an arrangement is being probed")
        return int(_probe_env.value_of(value))
    return int(value)


def _meta_operation(func):
    """On a tensor without a concrete shape (one written in a parameter annotation,
    ``tests/test_softmax.py:13-17``) the call is recorded and replayed when the front
    door probes the kernel; on a probe tensor it runs at once."""

    def wrapper(self, *args, **kwargs):
        if self._index is None:
            deferred = Tensor.__new__(Tensor)
            deferred.__dict__.update(self.__dict__)
            deferred._recorded = self._recorded + ((func.__name__, args, kwargs),)
            return deferred
        return func(self, *args, **kwargs)

    wrapper.__name__ = func.__name__
    wrapper.__doc__ = func.__doc__
    return wrapper


class Tensor:
    """A symbolic tensor.

    :param ndim: number of dimensions (0 for a scalar argument).
    :param shape: concrete or symbolic sizes (alternative to ``ndim``).
    :param dtype: element type tag (``ninetoothed_b200.float16`` ...), or, on an
        arranged tensor, the next level of the hierarchy.
    :param other: value read at masked positions (``float("-inf")`` for softmax).
    :param shape_options: per-dimension symbol options (``{"constexpr": True}``).
    :param constexpr: for 0-dim tensors: the value is a compile-time constant
        passed per call (``is_causal``).
    """

    num_instances = 0

    def __init__(self, ndim=None, shape=None, dtype=None, jagged_dim=None, other=None, shape_options=None,
                 constexpr=None, value=None, name=None):
        assert ndim is not None or shape is not None, "Either `ndim` or `shape` must be provided."
        if ndim is None:
            ndim = len(shape)
        if constexpr and ndim != 0:
            raise ValueError("`constexpr` can only be set for zero-dimensional tensors.")
        if not constexpr and value is not None:
            raise ValueError("`value` can only be set for constexpr tensors.")
        if jagged_dim is not None:
            raise NotImplementedError("jagged tensors are outside the kernels this library holds")
        self.spec_ndim = ndim
        self.spec_shape = tuple(shape) if shape is not None else tuple(None for _ in range(ndim))
        self.element_type = dtype
        self.other = other
        self.shape_options = shape_options
        self.constexpr = constexpr
        self.value = value
        self.name = name if name is not None else f"tensor_{type(self).num_instances}"
        type(self).num_instances += 1
        self.source = self
        # Probe state: filled by `instantiate`.
        self._index = None
        self._prefix = ()
        self._levels = None
        self._parent = None
        self._recorded = ()

    # -- probing ----------------------------------------------------------------
    def instantiate(self, shape):
        """A copy of this specification bound to a concrete shape, ready to be arranged."""
        bound = Tensor(self.spec_ndim, self.spec_shape, self.element_type, None, self.other, self.shape_options,
                       self.constexpr, self.value, self.name)
        shape = tuple(int(s) for s in shape)
        assert len(shape) == self.spec_ndim, (shape, self.spec_ndim)
        bound._index = np.arange(math.prod(shape), dtype=np.int64).reshape(shape)
        bound._levels = [shape]
        bound.source_shape = shape
        for name, args, kwargs in self._recorded:
            bound = getattr(bound, name)(*args, **kwargs)
        return bound

    def _derive(self, index, levels):
        out = Tensor.__new__(Tensor)
        out.__dict__.update(self.__dict__)
        out._index, out._levels = index, [tuple(level) for level in levels]
        out._parent = None
        return out

    @property
    def _p(self):
        return len(self._prefix)

    @property
    def ndim(self):
        return self.spec_ndim if self._levels is None else len(self._levels[0])

    @property
    def shape(self):
        if self._levels is None:
            return tuple(
                size if size is not None else Symbol(f"{self.name}_size_{i}")
                for i, size in enumerate(self.spec_shape)
            )
        return tuple(self._levels[0])

    @property
    def dtype(self):
        """Next level of an arranged tensor; the element type tag at the innermost level."""
        if self._levels is None or len(self._levels) == 1:
            return self.element_type
        inner = self._derive(self._index, self._levels[1:])
        inner._prefix = self._prefix + tuple(self._levels[0])
        inner._parent = self  # `x.dtype.dtype = ...` must reach x
        return inner

    @dtype.setter
    def dtype(self, value):
        if isinstance(value, Tensor) and value._index is not None and self._levels is not None:
            expected_prefix = self._prefix + tuple(self._levels[0])
            if tuple(value._prefix) != expected_prefix:
                raise ValueError("the assigned inner level does not belong under this tensor")
            self._index = value._index
            self._levels = [self._levels[0]] + list(value._levels)
            if self._parent is not None:
                self._parent.dtype = self
        else:
            self.element_type = value

    def levels(self):
        """Shapes of all levels, outermost first."""
        return [tuple(level) for level in self._levels]

    def index_map(self):
        """The index array: axes are the dimensions of every level, outermost first."""
        return self._index

    # -- meta-operations --------------------------------------------------------
    @_meta_operation
    def tile(self, tile_shape, strides=None, dilation=None, floor_mode=False):
        """Tiles the outermost level into (outer, tile) levels (``tensor.py:199-286``)."""
        shape = self._levels[0]
        if strides is None:
            strides = [-1] * len(tile_shape)
        if dilation is None:
            dilation = [1] * len(tile_shape)
        p, nd = self._p, len(shape)
        index = self._index
        outer_shape, inner_shape = [], []
        for dim, (size, tile_size, stride, spacing) in enumerate(zip(shape, tile_shape, strides, dilation)):
            tile_size, stride, spacing = _resolve(tile_size), _resolve(stride), _resolve(spacing)
            if tile_size == -1:
                tile_size = size
            if stride == -1:
                stride = tile_size
            span = size - spacing * (tile_size - 1) - 1
            if stride != 0:
                outer = (span // stride if floor_mode else -(-span // stride)) + 1
            else:
                outer = 1
            outer = max(outer, 0)
            outer_shape.append(outer)
            inner_shape.append(tile_size)
            positions = np.arange(outer)[:, None] * stride + np.arange(tile_size)[None, :] * spacing
            # positions outside [0, size) are masked: route them to an appended slab of -1
            axis = p + dim
            pad_shape = list(index.shape)
            pad_shape[axis] = 1
            padded = np.concatenate([index, np.full(pad_shape, -1, dtype=index.dtype)], axis=axis)
            safe = np.where((positions >= 0) & (positions < size), positions, size)
            gathered = np.take(padded, safe.reshape(-1), axis=axis)
            new_shape = list(index.shape)
            new_shape[axis:axis + 1] = [outer, tile_size]
            gathered = gathered.reshape(new_shape)
            # move the tile axis behind all remaining level-0 axes (it joins the inner level)
            inner_axis = axis + 1
            destination = p + nd + dim  # after the nd outer axes and the tile axes already moved
            index = np.moveaxis(gathered, inner_axis, destination)
        return self._derive(index, [outer_shape, inner_shape] + list(self._levels[1:]))

    @_meta_operation
    def expand(self, shape):
        """Broadcasts singleton dimensions of the outermost level (``tensor.py:288-321``)."""
        current = self._levels[0]
        new_level = [_resolve(new) if _resolve(new) != -1 else size for size, new in zip(current, shape)]
        target = list(self._index.shape)
        target[self._p:self._p + len(current)] = new_level
        index = np.broadcast_to(self._index, target)
        return self._derive(index, [new_level] + list(self._levels[1:]))

    @_meta_operation
    def unsqueeze(self, dim):
        """Inserts a singleton dimension (``tensor.py:323-354``)."""
        level = list(self._levels[0])
        dim = dim if dim >= 0 else dim + len(level) + 1
        level.insert(dim, 1)
        return self._derive(np.expand_dims(self._index, self._p + dim), [level] + list(self._levels[1:]))

    @_meta_operation
    def squeeze(self, dim):
        """Removes singleton dimensions (``tensor.py:356-394``)."""
        dims = dim if isinstance(dim, tuple) else (dim,)
        level = list(self._levels[0])
        dims = tuple(d if d >= 0 else d + len(level) for d in dims)
        for d in dims:
            if level[d] != 1:
                raise ValueError(f"cannot squeeze dimension {d} of size {level[d]}")
        index = np.squeeze(self._index, axis=tuple(self._p + d for d in dims))
        new_level = [size for i, size in enumerate(level) if i not in dims]
        return self._derive(index, [new_level] + list(self._levels[1:]))

    @_meta_operation
    def permute(self, dims):
        """Reorders the dimensions of the outermost level (``tensor.py:396-426``)."""
        level = self._levels[0]
        p = self._p
        axes = list(range(p)) + [p + d for d in dims] + list(range(p + len(level), self._index.ndim))
        return self._derive(np.transpose(self._index, axes), [[level[d] for d in dims]] + list(self._levels[1:]))

    @_meta_operation
    def flatten(self, start_dim=None, end_dim=None):
        """Merges dimensions [start_dim, end_dim) of the outermost level (``tensor.py:428-484``)."""
        level = list(self._levels[0])
        start = 0 if start_dim is None else (start_dim if start_dim >= 0 else start_dim + len(level))
        end = len(level) if end_dim is None else (end_dim if end_dim >= 0 else end_dim + len(level))
        new_level = level[:start] + [math.prod(level[start:end])] + level[end:]
        new_shape = list(self._index.shape)
        new_shape[self._p:self._p + len(level)] = new_level
        return self._derive(np.ascontiguousarray(self._index).reshape(new_shape), [new_level] + list(self._levels[1:]))

    @_meta_operation
    def ravel(self):
        """Collapses the hierarchy into one level (``tensor.py:486-541``)."""
        merged = [size for level in self._levels for size in level]
        return self._derive(self._index, [merged])

    @_meta_operation
    def pad(self, pad):
        """Adds masked borders around the outermost level (``tensor.py:543-569``)."""
        level = self._levels[0]
        widths = [(0, 0)] * self._p + [(_resolve(lo), _resolve(hi)) for lo, hi in pad]
        widths += [(0, 0)] * (self._index.ndim - len(widths))
        index = np.pad(self._index, widths, constant_values=-1)
        new_level = [size + _resolve(lo) + _resolve(hi) for size, (lo, hi) in zip(level, pad)]
        return self._derive(index, [new_level] + list(self._levels[1:]))
