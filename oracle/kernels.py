"""numpy restatement of the kernels the reference's definitions generate.

TEST INFRASTRUCTURE ONLY (see the package docstring).  Every function walks the
same blocks in the same order as the generated kernel and rounds where it
rounds.  Citations are paths inside the reference project.

Shared rules of the generated code that every function below honours:

* one program per outermost-level element of the first argument, unravelled
  row-major (``src/ninetoothed/generation.py:629-636, 676-706``);
* every load is masked by all index bounds, and masked lanes read 0 unless the
  tensor was declared with ``other=`` (``generation.py:638-645``; the
  interpreter fills zeros, ``triton/runtime/interpreter.py:449-455``);
* stores are masked the same way and cast implicitly to the output dtype.
"""

from __future__ import annotations

import math

import numpy as np

LOG2E = 1.44269504089  # the literal in tests/test_attention.py:46


def _ceil_div(a, b):
    return -(-a // b)


def _tile(x, r0, r1, c0, c1):
    """x[r0:r1, c0:c1] with out-of-range lanes reading 0 (masked load)."""
    out = np.zeros((r1 - r0, c1 - c0), dtype=x.dtype)
    rr1, cc1 = min(r1, x.shape[0]), min(c1, x.shape[1])
    if rr1 > r0 and cc1 > c0:
        out[: rr1 - r0, : cc1 - c0] = x[r0:rr1, c0:cc1]
    return out


def matmul_acc(lhs, rhs, block_m=64, block_n=64, block_k=64):
    """fp32 accumulators of the tiled dot loop, before the store.

    Follows ``tests/test_matmul.py:41-44`` (same loop as ``README.md:56-60``):
    ``acc = zeros(fp32); for k: acc += dot(lhs[k], rhs[k])`` per (BM, BN) output
    tile, tiles enumerated row-major (``tests/test_matmul.py:22-36``).  The dot
    takes the operands in their storage dtype and accumulates in fp32.
    """
    m, k = lhs.shape
    k2, n = rhs.shape
    assert k == k2
    acc = np.zeros((m, n), dtype=np.float32)
    for pm in range(_ceil_div(m, block_m)):
        for pn in range(_ceil_div(n, block_n)):
            r0, c0 = pm * block_m, pn * block_n
            t = np.zeros((block_m, block_n), dtype=np.float32)
            for kb in range(_ceil_div(k, block_k)):
                a = _tile(lhs, r0, r0 + block_m, kb * block_k, (kb + 1) * block_k)
                b = _tile(rhs, kb * block_k, (kb + 1) * block_k, c0, c0 + block_n)
                t = np.matmul(a, b, dtype=np.float32) + t
            r1, c1 = min(r0 + block_m, m), min(c0 + block_n, n)
            acc[r0:r1, c0:c1] = t[: r1 - r0, : c1 - c0]
    return acc


def matmul(lhs, rhs, out_dtype=np.float16, block_m=64, block_n=64, block_k=64):
    """``tests/test_matmul.py:41-45``: the accumulator is cast once at the store."""
    return matmul_acc(lhs, rhs, block_m, block_n, block_k).astype(out_dtype)


def bmm(lhs, rhs, out_dtype=np.float16, block_m=64, block_n=64, block_k=64):
    """The matmul of ``tests/test_matmul.py:41-45`` per leading batch index: lhs [B,M,K], rhs [B,K,N]
    (the batched matmul whose operand shapes ``docs/source/build.rst:237-245`` names)."""
    return np.stack([matmul(lhs[i], rhs[i], out_dtype, block_m, block_n, block_k) for i in range(lhs.shape[0])])


def addmm(input, mat1, mat2, beta, alpha, out_dtype=np.float16, block_m=64, block_n=64, block_k=64):
    """``tests/test_addmm.py:35-38``.

    The matmul application is inlined, including its ``.to(float16)`` store
    (``tests/test_matmul.py:45``), so the product is rounded to fp16 *before* the
    epilogue.  ``beta`` and ``alpha`` are 0-dim tensors, i.e. run-time scalars;
    Triton's promotion rule for scalar-times-tensor keeps the tensor's dtype, so
    ``beta * input + alpha * product`` is evaluated in the storage dtype with a
    rounding after each of the two products and after the sum (pinned by the
    golden vectors: an fp32 epilogue does not reproduce them).
    """
    dt = input.dtype
    prod = matmul_acc(mat1, mat2, block_m, block_n, block_k).astype(np.float16).astype(dt)
    beta_t, alpha_t = np.asarray(beta, dtype=dt), np.asarray(alpha, dtype=dt)
    out = (beta_t * input).astype(dt) + (alpha_t * prod).astype(dt)
    return out.astype(out_dtype)


def softmax(x, out_dtype=None):
    """``tests/test_softmax.py:18-21``: one program per row, whole row in a block.

    Lanes past the row end are loaded as -inf (``other=float("-inf")``,
    ``tests/test_softmax.py:15``) and so contribute exp(-inf)=0.  Math is fp32
    (the reference test is fp32-only; for fp16 storage the row is widened first).
    """
    out_dtype = out_dtype or x.dtype
    row = x.astype(np.float32)
    row_minus_max = row - row.max(axis=-1, keepdims=True)
    numerator = np.exp(row_minus_max)
    denominator = numerator.sum(axis=-1, keepdims=True, dtype=np.float32)
    return (numerator / denominator).astype(out_dtype)


def attention(q, k, v, is_causal, block_m=64, block_n=64, scale=None, out_dtype=None):
    """``tests/test_attention.py:45-70``, per (batch, head), KV tiles of ``block_n``.

    ``scale=None`` is the reference's own kernel: ``q * 1.44269504089`` is a
    tensor-times-literal product evaluated in the tensor's dtype (``:46``).  With
    a ``scale`` (the 0-dim run-time scalar of the scaled variant used for the
    1/sqrt(D) configuration) ``q * scale * 1.44269504089`` is two such products,
    each evaluated and rounded in the dtype of ``q`` (Triton keeps the tensor's
    dtype for scalar-times-tensor; pinned by the golden vectors).  Every KV tile
    is visited, also under the causal mask.
    ``block_m`` only groups independent rows and does not change any value.
    """
    out_dtype = out_dtype or v.dtype
    b, h, s, d = q.shape
    s_kv = k.shape[2]
    out = np.empty((b, h, s, d), dtype=out_dtype)
    n_tiles = _ceil_div(s_kv, block_n)
    s_pad = n_tiles * block_n
    rows = np.arange(s)[:, None]
    for bi in range(b):
        for hi in range(h):
            if scale is None:
                q_loaded = (q[bi, hi] * np.asarray(LOG2E, dtype=q.dtype)).astype(q.dtype)
            else:
                q_scaled = (q[bi, hi] * np.asarray(scale, dtype=q.dtype)).astype(q.dtype)
                q_loaded = (q_scaled * np.asarray(LOG2E, dtype=q.dtype)).astype(q.dtype)
            kp = np.zeros((s_pad, d), dtype=k.dtype)
            vp = np.zeros((s_pad, d), dtype=v.dtype)
            kp[:s_kv] = k[bi, hi]
            vp[:s_kv] = v[bi, hi]
            acc = np.zeros((s, d), dtype=np.float32)
            l_i = np.ones((s,), dtype=np.float32)
            m_i = np.full((s,), -np.inf, dtype=np.float32)
            for i in range(n_tiles):
                cols = np.arange(i * block_n, (i + 1) * block_n)[None, :]
                kt = kp[i * block_n : (i + 1) * block_n]
                vt = vp[i * block_n : (i + 1) * block_n]
                qk = np.matmul(q_loaded, kt.T, dtype=np.float32)
                qk = np.where(cols < s_kv, qk, -np.inf).astype(np.float32)
                if is_causal:
                    qk = np.where(rows >= cols, qk, -np.inf).astype(np.float32)
                m_ij = np.maximum(m_i, qk.max(axis=1))
                p = np.exp2(qk - m_ij[:, None])
                l_ij = p.sum(axis=1, dtype=np.float32)
                alpha = np.exp2(m_i - m_ij)
                acc = acc * alpha[:, None] + np.matmul(p.astype(v.dtype), vt, dtype=np.float32)
                m_i = m_ij
                l_i = l_i * alpha + l_ij
            out[bi, hi] = (acc / l_i[:, None]).astype(out_dtype)
    return out


def conv2d_im2col(x, r, s, pad_h, pad_w):
    """The arranged input of ``tests/test_conv2d.py:22-38``: A[(n,p,q),(c,r,s)].

    ``pad`` adds masked (zero) borders; ``tile((1,C,R,S), strides=(-1,-1,1,1))``
    slides an R x S window with stride 1; ``ravel``/``flatten`` order rows as
    (n, p, q) and columns as (c, r, s).
    """
    n, c, h, w = x.shape
    p = h + 2 * pad_h - r + 1
    q = w + 2 * pad_w - s + 1
    xp = np.zeros((n, c, h + 2 * pad_h, w + 2 * pad_w), dtype=x.dtype)
    xp[:, :, pad_h : pad_h + h, pad_w : pad_w + w] = x
    cols = np.empty((n, p, q, c, r, s), dtype=x.dtype)
    for ri in range(r):
        for si in range(s):
            cols[:, :, :, :, ri, si] = xp[:, :, ri : ri + p, si : si + q].transpose(0, 2, 3, 1)
    return cols.reshape(n * p * q, c * r * s), (n, p, q)


def conv2d(x, w, padding=(0, 0), out_dtype=None, block_m=64, block_n=64, block_k=64):
    """``tests/test_conv2d.py:13-48`` + the matmul application (``:106``).

    Implicit GEMM: A = im2col(x) [(n,p,q),(c,r,s)], B = w.flatten(1).T
    [(c,r,s),k], C = y.permute(0,2,3,1).flatten(0..2) [(n,p,q),k]; stride 1,
    dilation 1, no bias, K dimension walked in ``block_k`` chunks of (c,r,s).
    """
    out_dtype = out_dtype or x.dtype
    kout, c, r, s = w.shape
    a, (n, p, q) = conv2d_im2col(x, r, s, padding[0], padding[1])
    b = np.ascontiguousarray(w.reshape(kout, c * r * s).T)
    cmat = matmul_acc(a, b, block_m, block_n, block_k).astype(out_dtype)
    return np.ascontiguousarray(cmat.reshape(n, p, q, kout).transpose(0, 3, 1, 2))


# ---------------------------------------------------------------------------
# Seeded synthetic inputs shared by the golden generator, the tests and bench.
# numpy's PCG64 stream is stable across numpy releases, unlike device RNGs.
# ---------------------------------------------------------------------------

def normal(seed, shape, dtype=np.float16, scale=1.0, count=1):
    """``count`` arrays of ``scale * N(0,1)`` drawn in order from one seeded stream."""
    rng = np.random.default_rng(seed)
    arrays = [
        (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(dtype)
        for _ in range(count)
    ]
    return arrays[0] if count == 1 else arrays


def flops_matmul(m, n, k):
    return 2.0 * m * n * k


def flops_attention(b, h, s, d, is_causal):
    full = 4.0 * b * h * s * s * d
    return full / 2 if is_causal else full


def flops_conv2d(n, c, h, w, kout, r, s, pad_h, pad_w):
    p = h + 2 * pad_h - r + 1
    q = w + 2 * pad_w - s + 1
    return 2.0 * n * p * q * kout * c * r * s


def bytes_softmax(rows, cols, itemsize=2):
    return 2.0 * rows * cols * itemsize


def max_pool2d(x, window, ceil_mode=False):
    """``tests/test_max_pool2d.py:13-36``: non-overlapping ``window = (r, s)`` tiles of an NCHW tensor
    (stride = window), the maximum of each tile.  ``floor_mode=not ceil_mode`` on the tiling decides
    whether a ragged last tile exists (``:19-21``); positions outside the tensor are loaded as the
    input's ``other`` value, -inf (``:59``), so they never win.  max is exact in every dtype."""
    n, c, h, w = x.shape
    r, s = window
    div = (lambda a, b: -(-a // b)) if ceil_mode else (lambda a, b: a // b)
    p, q = div(h - r, r) + 1, div(w - s, s) + 1
    padded = np.full((n, c, p * r, q * s), -np.inf, dtype=np.float32)
    hh, ww = min(h, p * r), min(w, q * s)
    padded[:, :, :hh, :ww] = x[:, :, :hh, :ww].astype(np.float32)
    return padded.reshape(n, c, p, r, q, s).max(axis=(3, 5)).astype(x.dtype)


def default_scale(d):
    return 1.0 / math.sqrt(d)
