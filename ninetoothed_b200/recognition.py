"""Decides which hand-written kernel an (arrangement, application) pair denotes.

The reference compiles *any* pair into Triton source
(``src/ninetoothed/generation.py:46-133`` in the reference project).  This
library holds hand-written kernels for five pairs only, so the front door must
prove that the pair it was handed is one of them, and reject everything else
loudly (there is no generic fallback):

* the **arrangement** is run on probe tensors with small concrete shapes and its
  index maps (which source element every position of every tile reads, -1 where
  masked) are compared with the index maps of the kernel's own tiling, built here
  directly with numpy;
* the **application** is matched by the shape of its syntax tree: which
  ``ninetoothed.language`` functions it calls, in which order, around which loop.
"""

from __future__ import annotations

import ast
import inspect
import textwrap
from dataclasses import dataclass, field

import numpy as np

from ninetoothed_b200.tensor import ProbeScope, Tensor


class UnsupportedKernelError(NotImplementedError):
    """The pair is not one of the kernels this library implements."""


# ---------------------------------------------------------------------------
# Canonical index maps (numpy only; independent of the meta-operations)
# ---------------------------------------------------------------------------

def _ceil_div(a, b):
    return -(-a // b)


def _blocked(matrix_index, block_rows, block_cols):
    """[R, C] index matrix -> [nR, nC, block_rows, block_cols], -1 outside."""
    rows, cols = matrix_index.shape
    n_r, n_c = _ceil_div(rows, block_rows), _ceil_div(cols, block_cols)
    padded = np.full((n_r * block_rows, n_c * block_cols), -1, dtype=np.int64)
    padded[:rows, :cols] = matrix_index
    return padded.reshape(n_r, block_rows, n_c, block_cols).transpose(0, 2, 1, 3)


def matmul_maps(a_index, b_index, c_index, bm, bn, bk):
    """Index maps of the tiled matmul (``tests/test_matmul.py:14-38``) over index
    matrices A [M,K], B [K,N], C [M,N] (identity maps for a plain matmul, im2col
    maps for conv2d)."""
    a_blocks = _blocked(a_index, bm, bk)  # [nM, nK, bm, bk]
    b_blocks = _blocked(b_index, bk, bn)  # [nK, nN, bk, bn]
    c_blocks = _blocked(c_index, bm, bn)  # [nM, nN, bm, bn]
    n_m, n_k = a_blocks.shape[:2]
    n_n = b_blocks.shape[1]
    a_map = np.broadcast_to(a_blocks[:, None], (n_m, n_n, n_k, bm, bk))
    b_map = np.broadcast_to(b_blocks.transpose(1, 0, 2, 3)[None], (n_m, n_n, n_k, bk, bn))
    return a_map, b_map, c_blocks


def identity(shape):
    return np.arange(int(np.prod(shape)), dtype=np.int64).reshape(shape)


def softmax_map(rows, cols, block):
    """``Tensor(2).tile((1, BLOCK))`` (``tests/test_softmax.py:15-16``): [rows, nblk, 1, BLOCK]."""
    return _blocked(identity((rows, cols)), 1, block)


def attention_maps(shape, bm, bn):
    """``tests/test_attention.py:14-42``: q/o [B,H,nQ,1,bm,D]; k/v [B,H,nQ,1,nKV,bn,D]."""
    b, h, s, d = shape
    src = identity(shape)
    n_q, n_kv = _ceil_div(s, bm), _ceil_div(s, bn)
    q_pad = np.full((b, h, n_q * bm, d), -1, dtype=np.int64)
    q_pad[:, :, :s] = src
    q_map = q_pad.reshape(b, h, n_q, bm, d)[:, :, :, None]
    kv_pad = np.full((b, h, n_kv * bn, d), -1, dtype=np.int64)
    kv_pad[:, :, :s] = src
    kv_blocks = kv_pad.reshape(b, h, n_kv, bn, d)
    kv_map = np.broadcast_to(kv_blocks[:, :, None, None], (b, h, n_q, 1, n_kv, bn, d))
    return q_map, kv_map


def conv2d_index_matrices(xshape, wshape, pad_h, pad_w):
    """im2col views of ``tests/test_conv2d.py:22-41``: A[(n,p,q),(c,r,s)], B[(c,r,s),k], C[(n,p,q),k]."""
    n, c, h, w = xshape
    k, _, r, s = wshape
    p, q = h + 2 * pad_h - r + 1, w + 2 * pad_w - s + 1
    x_pad = np.pad(identity(xshape), ((0, 0), (0, 0), (pad_h, pad_h), (pad_w, pad_w)), constant_values=-1)
    a = np.empty((n, p, q, c, r, s), dtype=np.int64)
    for ri in range(r):
        for si in range(s):
            a[:, :, :, :, ri, si] = x_pad[:, :, ri:ri + p, si:si + q].transpose(0, 2, 3, 1)
    a = a.reshape(n * p * q, c * r * s)
    b = identity(wshape).reshape(k, c * r * s).T
    cmat = identity((n, k, p, q)).transpose(0, 2, 3, 1).reshape(n * p * q, k)
    return a, b, cmat, (p, q)


def max_pool2d_maps(xshape, window, ceil_mode, block):
    """``tests/test_max_pool2d.py:13-33``: input [nB, 1, block, r*s] (the windows of ``block``
    consecutive outputs, -1 outside the tensor), output [nB, 1, block] (the outputs themselves)."""
    n, c, h, w = xshape
    r, s = window
    div = (lambda a, b: -(-a // b)) if ceil_mode else (lambda a, b: a // b)
    p, q = div(h - r, r) + 1, div(w - s, s) + 1
    x_pad = np.full((n, c, p * r, q * s), -1, dtype=np.int64)
    hh, ww = min(h, p * r), min(w, q * s)
    x_pad[:, :, :hh, :ww] = identity(xshape)[:, :, :hh, :ww]
    windows = x_pad.reshape(n, c, p, r, q, s).transpose(0, 1, 2, 4, 3, 5).reshape(n * c * p * q, r * s)
    outputs = identity((n, c, p, q)).reshape(n * c * p * q, 1)
    return _blocked(windows, block, r * s), _blocked(outputs, block, 1)[..., 0], (p, q)


# ---------------------------------------------------------------------------
# Arrangement probing
# ---------------------------------------------------------------------------

@dataclass
class Recognised:
    op: str                                   # matmul | addmm | softmax | attention | attention_scaled | conv2d | max_pool2d
    constexpr_names: tuple = ()               # per-call keyword arguments, sorted (bare names)
    block_sizes: dict = field(default_factory=dict)
    padded: bool = False                      # conv2d: arrangement pads with padding_h/padding_w symbols
    ceil_mode: bool = False                   # max_pool2d: the tiling keeps a ragged last window


def _is_arranged(x):
    return isinstance(x, Tensor) and x.index_map() is not None


def _same(a, b):
    return a.shape == b.shape and np.array_equal(a, b)


def _run(arrangement, specs, shapes, env=None):
    """Arrange probe tensors; returns (results, scope)."""
    with ProbeScope(env) as scope:
        # `instantiate` replays meta-operations recorded on annotation-style tensors,
        # which may name symbols, so it runs inside the scope too
        bound = [spec.instantiate(shape) if shape is not None else spec for spec, shape in zip(specs, shapes)]
        out = arrangement(*bound)
    return (out if isinstance(out, tuple) else (out,)), scope


def _check_matmul_like(arranged, a_index, b_index, c_index, extra_c=None):
    """arranged = (A, B, C[, C2]) probe results; verify against the canonical tiling."""
    a, b, c = arranged[:3]
    if not all(_is_arranged(t) for t in (a, b, c)):
        return None
    la, lb, lc = a.levels(), b.levels(), c.levels()
    if len(la) != 3 or len(lb) != 3 or len(lc) != 2 or len(la[2]) != 2 or len(lb[2]) != 2 or len(lc[1]) != 2:
        return None
    (bm, bk), (bk2, bn) = la[2], lb[2]
    if bk != bk2 or tuple(lc[1]) != (bm, bn):
        return None
    a_map, b_map, c_map = matmul_maps(a_index, b_index, c_index, bm, bn, bk)
    if not (_same(a.index_map(), a_map) and _same(b.index_map(), b_map) and _same(c.index_map(), c_map)):
        return None
    if extra_c is not None and not (_is_arranged(extra_c) and _same(extra_c.index_map(), c_map)):
        return None
    return {"BLOCK_SIZE_M": bm, "BLOCK_SIZE_N": bn, "BLOCK_SIZE_K": bk}


def _constexpr_names(scope):
    return tuple(sorted(s.name for s in scope.used if s.constexpr and not s.meta))


def recognise_arrangement(arrangement, specs):
    """Which kernel's tiling ``arrangement`` produces for the tensor ``specs``."""
    ndims = tuple(spec.spec_ndim for spec in specs)
    flags = tuple(bool(spec.constexpr) for spec in specs)
    try:
        if ndims == (2, 2, 2):
            m, n, k = 5, 7, 6
            out, scope = _run(arrangement, specs, [(m, k), (k, n), (m, n)])
            blocks = _check_matmul_like(out, identity((m, k)), identity((k, n)), identity((m, n)))
            if blocks and len(out) == 3:
                return Recognised("matmul", _constexpr_names(scope), blocks)
        elif ndims == (2, 2, 2, 0, 0, 2) and not any(flags):
            m, n, k = 5, 7, 6
            out, scope = _run(arrangement, specs, [(m, n), (m, k), (k, n), None, None, (m, n)])
            if len(out) == 6 and out[3] is specs[3] and out[4] is specs[4]:
                blocks = _check_matmul_like((out[1], out[2], out[5]), identity((m, k)), identity((k, n)),
                                            identity((m, n)), extra_c=out[0])
                if blocks:
                    return Recognised("addmm", _constexpr_names(scope), blocks)
        elif ndims == (4, 4):
            xshape, window, block = (2, 3, 7, 8), (3, 2), 4
            for ceil_mode in (False, True):
                in_map, out_map, (p, q) = max_pool2d_maps(xshape, window, ceil_mode, block)
                out, scope = _run(arrangement, specs, [xshape, (xshape[0], xshape[1], p, q)],
                                  env={"WINDOW_HEIGHT": window[0], "WINDOW_WIDTH": window[1], "BLOCK_SIZE": block})
                if len(out) == 2 and all(_is_arranged(t) for t in out) and _same(out[0].index_map(), in_map) \
                        and _same(out[1].index_map(), out_map):
                    names = _constexpr_names(scope)
                    if set(names) != {"WINDOW_HEIGHT", "WINDOW_WIDTH"}:
                        continue
                    if specs[0].other not in (float("-inf"),):
                        raise UnsupportedKernelError(
                            "max_pool2d: the input must be declared with other=float('-inf') so that positions "
                            "outside the tensor never win the maximum"
                        )
                    return Recognised("max_pool2d", names, {"BLOCK_SIZE": block}, ceil_mode=ceil_mode)
        elif ndims == (2, 2):
            rows, cols = 5, 7
            out, scope = _run(arrangement, specs, [(rows, cols), (rows, cols)], env={"BLOCK_SIZE": 8})
            if len(out) == 2 and all(_is_arranged(t) for t in out) and len(out[0].levels()) == 2:
                block = out[0].levels()[1][-1]
                expected = softmax_map(rows, cols, block)
                if block >= cols and _same(out[0].index_map(), expected) and _same(out[1].index_map(), expected):
                    if specs[0].other not in (float("-inf"),):
                        raise UnsupportedKernelError(
                            "softmax: the input must be declared with other=float('-inf') so that lanes past the "
                            "row end do not take part in the row maximum and sum"
                        )
                    return Recognised("softmax", _constexpr_names(scope), {"BLOCK_SIZE": block})
        elif ndims in ((4, 4, 4, 0, 4), (4, 4, 4, 0, 0, 4)):
            scaled = len(ndims) == 6
            causal_at = 4 if scaled else 3
            if flags[causal_at] and not (scaled and flags[3]):
                shape = (2, 3, 7, 4)
                shapes = [shape] * 3 + [None] * (2 if scaled else 1) + [shape]
                out, scope = _run(arrangement, specs, shapes)
                passthrough = all(out[i] is specs[i] for i in range(3, causal_at + 1))
                tensors = (out[0], out[1], out[2], out[-1])
                if len(out) == len(specs) and passthrough and all(_is_arranged(t) for t in tensors):
                    lq, lk = out[0].levels(), out[1].levels()
                    if len(lq) == 2 and len(lk) == 3 and len(lq[1]) == 2 and len(lk[2]) == 2:
                        bm, bn = lq[1][0], lk[2][0]
                        q_map, kv_map = attention_maps(shape, bm, bn)
                        if (_same(out[0].index_map(), q_map) and _same(out[-1].index_map(), q_map)
                                and _same(out[1].index_map(), kv_map) and _same(out[2].index_map(), kv_map)):
                            return Recognised("attention_scaled" if scaled else "attention", _constexpr_names(scope),
                                              {"BLOCK_SIZE_M": bm, "BLOCK_SIZE_N": bn})
        elif ndims == (4, 4, 4):
            xshape, wshape = (2, 3, 5, 6), (4, 3, 3, 2)
            for pad_h, pad_w, padded in ((1, 2, True), (0, 0, False)):
                a, b, c, (p, q) = conv2d_index_matrices(xshape, wshape, pad_h, pad_w)
                yshape = (xshape[0], wshape[0], p, q)
                out, scope = _run(arrangement, specs, [xshape, wshape, yshape],
                                  env={"padding_h": pad_h, "padding_w": pad_w})
                names = _constexpr_names(scope)
                uses_padding = {"padding_h", "padding_w"} <= set(names)
                if uses_padding != padded:
                    continue
                blocks = _check_matmul_like(out, a, b, c)
                if blocks and len(out) == 3:
                    return Recognised("conv2d", names, blocks, padded=padded)
    except UnsupportedKernelError:
        raise
    except Exception as error:  # the arrangement used something the probe cannot follow
        raise UnsupportedKernelError(
            f"the arrangement could not be evaluated on probe tensors ({type(error).__name__}: {error})"
        ) from error
    raise UnsupportedKernelError(
        f"no hand-written kernel matches this arrangement (tensor ranks {ndims}); this library implements the "
        "matmul, addmm, row-softmax, attention, conv2d and max_pool2d arrangements only and has no generic code generator"
    )


# ---------------------------------------------------------------------------
# Application fingerprints
# ---------------------------------------------------------------------------

class _CallCollector(ast.NodeVisitor):
    """Collects, in source order, the names of ``<language alias>.<fn>(...)`` and
    ``<expr>.to(...)`` calls, inlining calls to other Python functions the way the
    reference's inliner does (``src/ninetoothed/generation.py:884-1114``)."""

    def __init__(self, func):
        self.calls = []
        self.loops = 0
        self.branches = 0
        self.constants = []
        self.binops = []
        self._globals = getattr(func, "__globals__", {})
        self._language_aliases = {
            name for name, value in self._globals.items()
            if getattr(value, "__name__", "") in ("ninetoothed_b200.language", "ninetoothed.language")
        }
        self._depth = 0

    def visit_For(self, node):
        self.loops += 1
        self.generic_visit(node)

    def visit_If(self, node):
        self.branches += 1
        self.generic_visit(node)

    def visit_Constant(self, node):
        if isinstance(node.value, float):
            self.constants.append(node.value)

    def visit_BinOp(self, node):
        self.binops.append(type(node.op).__name__)
        self.generic_visit(node)

    def visit_AugAssign(self, node):
        self.binops.append("Aug" + type(node.op).__name__)
        self.generic_visit(node)

    def _resolve(self, node):
        if isinstance(node, ast.Name):
            return self._globals.get(node.id)
        if isinstance(node, ast.Attribute):
            base = self._resolve(node.value)
            return getattr(base, node.attr, None) if base is not None else None
        return None

    def visit_Call(self, node):
        func = node.func
        if isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name) \
                and func.value.id in self._language_aliases:
            self.generic_visit(node)
            self.calls.append(func.attr)
            return
        if isinstance(func, ast.Attribute) and func.attr in ("to", "offsets"):
            self.generic_visit(node)
            self.calls.append("." + func.attr)
            return
        if isinstance(func, ast.Name) and func.id in ("range", "float", "int", "bool", "len", "min", "max"):
            self.generic_visit(node)
            return
        target = self._resolve(func)
        if inspect.isfunction(target) and self._depth < 4:
            for arg in node.args:
                self.visit(arg)
            inner = _CallCollector(target)
            inner._depth = self._depth + 1
            inner.visit(_parse(target))
            self.calls.extend(inner.calls)
            self.loops += inner.loops
            self.branches += inner.branches
            self.constants.extend(inner.constants)
            self.binops.extend(inner.binops)
            return
        self.generic_visit(node)
        self.calls.append("?")


def _parse(func):
    try:
        source = textwrap.dedent(inspect.getsource(func))
    except (OSError, TypeError) as error:
        raise UnsupportedKernelError(
            f"the source of {getattr(func, '__name__', func)!r} is not available, so the application cannot be "
            "recognised"
        ) from error
    tree = ast.parse(source)
    return tree.body[0]


def fingerprint(application):
    node = _parse(application)
    collector = _CallCollector(application)
    for statement in node.body:
        collector.visit(statement)
    return collector


def _without(calls, *names):
    return [c for c in calls if c not in names]


def recognise_application(application):
    """matmul | addmm | softmax | attention | attention_scaled | row_max, from the syntax tree."""
    fp = fingerprint(application)
    calls = fp.calls
    n_params = len(inspect.signature(application).parameters)
    core = _without(calls, ".to")
    if core == ["zeros", "dot"] and fp.loops == 1 and n_params == 3 and "AugAdd" in fp.binops:
        return "matmul"
    if core == ["zeros", "zeros", "dot"] and fp.loops == 1 and n_params == 6 \
            and fp.binops.count("Mult") == 2 and "Add" in fp.binops:
        return "addmm"
    if core == ["max", "exp", "sum"] and fp.loops == 0 and n_params == 2 \
            and "Sub" in fp.binops and "Div" in fp.binops:
        return "softmax"
    if calls == ["max"] and fp.loops == 0 and fp.branches == 0 and n_params == 2 and not fp.binops:
        return "row_max"
    attention_core = _without(core, ".offsets")
    expected = ["zeros", "full", "full", "trans", "dot", "where", "where", "max", "maximum", "exp2", "sum", "exp2",
                "dot"]
    if attention_core == expected and fp.loops == 1 and fp.branches == 1 \
            and any(abs(c - 1.44269504089) < 1e-9 for c in fp.constants):
        if n_params == 5 and fp.binops.count("Mult") == 3:
            return "attention"
        if n_params == 6 and fp.binops.count("Mult") == 4:
            return "attention_scaled"
    raise UnsupportedKernelError(
        f"no hand-written kernel matches this application (language calls {calls}); this library implements the "
        "matmul, addmm, row-softmax, attention and window-maximum applications only and has no generic code generator"
    )


def recognise(arrangement, application, specs):
    arranged = recognise_arrangement(arrangement, specs)
    applied = recognise_application(application)
    compatible = {
        "matmul": {"matmul"},
        "addmm": {"addmm"},
        "softmax": {"softmax"},
        "attention": {"attention"},
        "attention_scaled": {"attention_scaled"},
        "conv2d": {"matmul"},  # conv2d is the im2col arrangement under the matmul application
        "max_pool2d": {"row_max"},  # max_pool2d is the window arrangement under a maximum along axis 1
    }
    if applied not in compatible[arranged.op]:
        raise UnsupportedKernelError(
            f"the arrangement tiles like {arranged.op} but the application computes {applied}"
        )
    return arranged
