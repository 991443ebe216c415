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
* the **application** must equal, statement by statement (up to the names of
  variables), one of the bodies the kernels implement.
"""

from __future__ import annotations

import ast
import copy
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


def bmm_maps(batch, m, n, k, bm, bn, bk):
    """The matmul tiling under a leading batch dimension of tile size 1: A [B,nM,nN,nK,bm,bk],
    B [B,nM,nN,nK,bk,bn], C [B,nM,nN,bm,bn]."""
    a, b, c = identity((batch, m, k)), identity((batch, k, n)), identity((batch, m, n))
    per_batch = [matmul_maps(a[i], b[i], c[i], bm, bn, bk) for i in range(batch)]
    return tuple(np.stack([maps[which] for maps in per_batch]) for which in range(3))


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
    op: str                                   # matmul | bmm | addmm | softmax | attention | attention_scaled | conv2d | max_pool2d
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
        elif ndims == (3, 3, 3):
            batch, m, n, k = 2, 5, 7, 6
            out, scope = _run(arrangement, specs, [(batch, m, k), (batch, k, n), (batch, m, n)])
            if len(out) == 3 and all(_is_arranged(t) for t in out):
                la, lb, lc = (t.levels() for t in out)
                if len(la) == 3 and len(lb) == 3 and len(lc) == 2 and len(la[2]) == 2 and len(lb[2]) == 2 \
                        and len(lc[1]) == 2:
                    (bm, bk), (bk2, bn) = la[2], lb[2]
                    if bk == bk2 and tuple(lc[1]) == (bm, bn):
                        a_map, b_map, c_map = bmm_maps(batch, m, n, k, bm, bn, bk)
                        if _same(out[0].index_map(), a_map) and _same(out[1].index_map(), b_map) \
                                and _same(out[2].index_map(), c_map):
                            return Recognised("bmm", _constexpr_names(scope),
                                              {"BLOCK_SIZE_M": bm, "BLOCK_SIZE_N": bn, "BLOCK_SIZE_K": bk})
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
# Application matching: the whole body, statement by statement
# ---------------------------------------------------------------------------
# A hand-written kernel computes exactly one thing, so an application is accepted only when
# its body IS one of the bodies below: same statements, same operators and operand order, same
# language calls with the same arguments, no extra constants.  What may differ is what cannot
# change the result: the names of parameters and local variables, the alias under which
# ``ninetoothed.language`` was imported, comments and docstrings, and whether a helper
# application is called or written out (calls to other Python functions are inlined the way the
# reference's inliner does, ``src/ninetoothed/generation.py:884-1114`` in the reference project).
# A cast to ``float16`` or ``bfloat16`` names the storage type: the kernels round to the dtype
# of the output tensor, so the two spellings are one.

_CANONICAL_SOURCES = {
    # tests/test_matmul.py:41-45, and README.md:55-61 (no cast: the store rounds)
    "matmul": ("""
def application(lhs, rhs, output):
    accumulator = ntl.zeros(output.shape, dtype=ntl.float32)
    for k in range(lhs.shape[0]):
        accumulator += ntl.dot(lhs[k], rhs[k])
    output = accumulator.to(ntl.float16)
""", """
def application(input, other, output):
    accumulator = ntl.zeros(output.shape, dtype=ntl.float32)
    for k in range(input.shape[0]):
        accumulator += ntl.dot(input[k], other[k])
    output = accumulator
"""),
    # tests/test_addmm.py:35-38 with the matmul application written out
    "addmm": ("""
def application(input, mat1, mat2, beta, alpha, output):
    matmul_output = ntl.zeros(output.shape, dtype=ntl.float32)
    accumulator = ntl.zeros(matmul_output.shape, dtype=ntl.float32)
    for k in range(mat1.shape[0]):
        accumulator += ntl.dot(mat1[k], mat2[k])
    matmul_output = accumulator.to(ntl.float16)
    output = beta * input + alpha * matmul_output
""",),
    # tests/test_softmax.py:18-21, and the same with the row widened to fp32 first
    "softmax": ("""
def application(input_row, output_row):
    row_minus_max = input_row - ntl.max(input_row)
    numerator = ntl.exp(row_minus_max)
    denominator = ntl.sum(numerator)
    output_row = numerator / denominator
""", """
def application(input_row, output_row):
    loaded = input_row
    row = loaded.to(ntl.float32)
    row_minus_max = row - ntl.max(row)
    numerator = ntl.exp(row_minus_max)
    denominator = ntl.sum(numerator)
    output_row = numerator / denominator
"""),
    # tests/test_max_pool2d.py:35-36
    "row_max": ("""
def application(input, output):
    output = ntl.max(input, axis=1)
""",),
}

# tests/test_attention.py:45-70; the scaled form multiplies q by one more scalar before log2(e)
_ATTENTION_BODY = """
    acc = ntl.zeros((q.shape[-2], q.shape[-1]), dtype=ntl.float32)
    l_i = ntl.full((q.shape[-2],), 1, dtype=ntl.float32)
    m_i = ntl.full((q.shape[-2],), float("-inf"), dtype=ntl.float32)
    for i in range(k.shape[0]):
        qk = ntl.dot(q_loaded, ntl.trans(k[i]))
        qk = ntl.where(k[i].offsets(-2) < k.source.shape[-2], qk, float("-inf"))
        if is_causal:
            mask = q.offsets(-2)[:, None] >= k[i].offsets(-2)[None, :]
            qk = ntl.where(mask, qk, float("-inf"))
        m_ij = ntl.maximum(m_i, ntl.max(qk, 1))
        p = ntl.exp2(qk - m_ij[:, None])
        l_ij = ntl.sum(p, 1)
        alpha = ntl.exp2(m_i - m_ij)
        acc = acc * alpha[:, None] + ntl.dot(p.to(v[i].dtype), v[i])
        m_i = m_ij
        l_i = l_i * alpha + l_ij
    acc /= l_i[:, None]
    o = acc
"""
_CANONICAL_SOURCES["attention"] = (
    "\ndef application(q, k, v, is_causal, o):\n    q_loaded = (q * 1.44269504089).to(q.dtype)\n" + _ATTENTION_BODY,)
_CANONICAL_SOURCES["attention_scaled"] = (
    "\ndef application(q, k, v, scale, is_causal, o):\n    q_loaded = (q * scale * 1.44269504089).to(q.dtype)\n"
    + _ATTENTION_BODY,)

_LANGUAGE_MODULES = ("ninetoothed_b200.language", "ninetoothed.language")
_MAX_INLINE_DEPTH = 4


def _parse(func):
    try:
        source = textwrap.dedent(inspect.getsource(func))
    except (OSError, TypeError) as error:
        raise UnsupportedKernelError(
            f"the source of {getattr(func, '__name__', func)!r} is not available, so the application cannot be "
            "recognised"
        ) from error
    return ast.parse(source).body[0]


def _resolve(node, namespace):
    if isinstance(node, ast.Name):
        return namespace.get(node.id)
    if isinstance(node, ast.Attribute):
        base = _resolve(node.value, namespace)
        return getattr(base, node.attr, None) if base is not None else None
    return None


class _Substitute(ast.NodeTransformer):
    """Replaces names: callee parameters by the caller's argument expressions, callee locals by fresh names."""

    def __init__(self, mapping):
        self.mapping = mapping

    def visit_Name(self, node):
        replacement = self.mapping.get(node.id)
        if replacement is None:
            return node
        if isinstance(replacement, ast.Name):
            return ast.copy_location(ast.Name(id=replacement.id, ctx=node.ctx), node)
        if not isinstance(node.ctx, ast.Load):
            raise UnsupportedKernelError("an inlined application assigns to a parameter that was passed an expression")
        return copy.deepcopy(replacement)


def _assigned_names(statements):
    names = []
    for statement in statements:
        for node in ast.walk(statement):
            if isinstance(node, ast.Name) and isinstance(node.ctx, ast.Store) and node.id not in names:
                names.append(node.id)
    return names


def _language_aliases(namespace):
    return {name for name, value in namespace.items() if getattr(value, "__name__", "") in _LANGUAGE_MODULES}


def _inlined_body(func_def, namespace, depth, counter):
    """The statements of ``func_def`` with statement-level calls to Python functions written out."""
    body = []
    aliases = _language_aliases(namespace)
    for statement in func_def.body:
        if isinstance(statement, ast.Expr) and isinstance(statement.value, ast.Constant) \
                and isinstance(statement.value.value, str):
            continue  # a docstring
        call = statement.value if isinstance(statement, ast.Expr) else None
        target = _resolve(call.func, namespace) if isinstance(call, ast.Call) else None
        if not inspect.isfunction(target):
            body.append(statement)
            continue
        if depth >= _MAX_INLINE_DEPTH or call.keywords:
            raise UnsupportedKernelError("calls between applications nest too deeply or use keyword arguments")
        callee = _parse(target)
        parameters = [a.arg for a in callee.args.args]
        if len(parameters) != len(call.args):
            raise UnsupportedKernelError(f"{target.__name__}() is called with the wrong number of arguments")
        callee_namespace = getattr(target, "__globals__", {})
        inner = _inlined_body(callee, callee_namespace, depth + 1, counter)
        mapping = dict(zip(parameters, call.args))
        counter[0] += 1
        for name in _assigned_names(inner):
            if name not in mapping:
                mapping[name] = ast.Name(id=f"{name}__inlined{counter[0]}", ctx=ast.Load())
        # the callee's alias of the language module becomes the caller's
        caller_alias = sorted(aliases)[0] if aliases else None
        for alias in _language_aliases(callee_namespace):
            if caller_alias is not None and alias not in mapping:
                mapping[alias] = ast.Name(id=caller_alias, ctx=ast.Load())
        substitute = _Substitute(mapping)
        body.extend(substitute.visit(copy.deepcopy(s)) for s in inner)
    return body


class _Normalise(ast.NodeTransformer):
    """Parameters -> a0, a1, ...; locals -> v0, v1, ... in order of appearance; the language alias -> ntl."""

    def __init__(self, parameters, local_names, aliases):
        self.names = {name: f"a{i}" for i, name in enumerate(parameters)}
        self.local_names = set(local_names)
        self.aliases = aliases
        self.count = 0

    def visit_Name(self, node):
        if node.id in self.aliases and node.id not in self.names:
            return ast.copy_location(ast.Name(id="ntl", ctx=node.ctx), node)
        if node.id not in self.names and node.id in self.local_names:
            self.names[node.id] = f"v{self.count}"
            self.count += 1
        return ast.copy_location(ast.Name(id=self.names.get(node.id, node.id), ctx=node.ctx), node)

    def visit_Attribute(self, node):
        node = self.generic_visit(node)
        if isinstance(node.value, ast.Name) and node.value.id == "ntl" and node.attr == "bfloat16":
            node.attr = "float16"  # either spelling names the 16-bit storage type
        return node


def canonical_text(func_def, namespace):
    """Normalised text of an application body (see the comment above ``_CANONICAL_SOURCES``)."""
    parameters = [a.arg for a in func_def.args.args]
    body = _inlined_body(func_def, namespace, 0, [0])
    normalise = _Normalise(parameters, _assigned_names(body), _language_aliases(namespace))
    module = ast.Module(body=[normalise.visit(copy.deepcopy(s)) for s in body], type_ignores=[])
    return f"{len(parameters)} parameters\n" + ast.unparse(ast.fix_missing_locations(module))


def _canonical_table():
    table = {}
    namespace = {"ntl": type("language", (), {"__name__": _LANGUAGE_MODULES[0]})()}
    for op, sources in _CANONICAL_SOURCES.items():
        for source in sources:
            table[canonical_text(ast.parse(textwrap.dedent(source)).body[0], namespace)] = op
    return table


_CANONICAL = _canonical_table()


def recognise_application(application):
    """matmul | addmm | softmax | attention | attention_scaled | row_max: the body must equal, statement by
    statement, one of the bodies this library implements."""
    text = canonical_text(_parse(application), getattr(application, "__globals__", {}))
    op = _CANONICAL.get(text)
    if op is None:
        raise UnsupportedKernelError(
            f"no hand-written kernel matches the application {getattr(application, '__name__', application)!r}: "
            "its body is not, statement by statement, one of the matmul, addmm, row-softmax, attention or "
            "window-maximum bodies this library implements (there is no generic code generator).  Normalised body:\n"
            + text
        )
    return op


def recognise(arrangement, application, specs):
    arranged = recognise_arrangement(arrangement, specs)
    applied = recognise_application(application)
    compatible = {
        "matmul": {"matmul"},
        "bmm": {"matmul"},  # the matmul application under a leading batch dimension
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
