"""The kernels as a user of the arrange-and-apply API writes them.

These are the definitions the reference's own tests use (matmul:
tests/test_matmul.py:14-45, addmm: tests/test_addmm.py:13-38, softmax:
tests/test_softmax.py:10-27, attention: tests/test_attention.py:14-70, conv2d:
tests/test_conv2d.py:13-48, max_pool2d: tests/test_max_pool2d.py:13-36 in the reference project).
They are user code, not part of the library: the tests, the benchmark and the smoke
test go through them.

The text is written against a front end called ``ninetoothed``.  Imported normally the
module binds that name to ``ninetoothed_b200``; ``examples.load_definitions("ninetoothed")``
executes the same text against the reference package instead, which is how the same
definitions are run through the reference's Triton back end for comparison.
"""

import functools
import importlib

ninetoothed = importlib.import_module(globals().get("__front_end__", "ninetoothed_b200"))
ntl = importlib.import_module(ninetoothed.__name__ + ".language")
Symbol, Tensor, block_size = ninetoothed.Symbol, ninetoothed.Tensor, ninetoothed.block_size

BLOCK_SIZE_M = Symbol("BLOCK_SIZE_M", meta=True)
BLOCK_SIZE_N = Symbol("BLOCK_SIZE_N", meta=True)
BLOCK_SIZE_K = Symbol("BLOCK_SIZE_K", meta=True)


# ------------------------------------------------------------------ matmul
def matmul_arrangement(lhs, rhs, output, BLOCK_SIZE_M=BLOCK_SIZE_M, BLOCK_SIZE_N=BLOCK_SIZE_N,
                       BLOCK_SIZE_K=BLOCK_SIZE_K):
    output_tiled = output.tile((BLOCK_SIZE_M, BLOCK_SIZE_N))

    lhs_tiled = lhs.tile((BLOCK_SIZE_M, BLOCK_SIZE_K)).tile((1, -1)).expand((-1, output_tiled.shape[1]))
    lhs_tiled.dtype = lhs_tiled.dtype.squeeze(0)

    rhs_tiled = rhs.tile((BLOCK_SIZE_K, BLOCK_SIZE_N)).tile((-1, 1)).expand((output_tiled.shape[0], -1))
    rhs_tiled.dtype = rhs_tiled.dtype.squeeze(1)

    return lhs_tiled, rhs_tiled, output_tiled


def matmul_application(lhs, rhs, output):
    accumulator = ntl.zeros(output.shape, dtype=ntl.float32)
    for k in range(lhs.shape[0]):
        accumulator += ntl.dot(lhs[k], rhs[k])
    output = accumulator.to(ntl.float16)  # noqa: F841


def readme_matmul_application(input, other, output):
    accumulator = ntl.zeros(output.shape, dtype=ntl.float32)

    for k in range(input.shape[0]):
        accumulator += ntl.dot(input[k], other[k])

    output = accumulator  # noqa: F841


def make_matmul(**kwargs):
    return ninetoothed.make(matmul_arrangement, matmul_application, (Tensor(2), Tensor(2), Tensor(2)), **kwargs)


# --------------------------------------------------------------------- bmm
def bmm_arrangement(lhs, rhs, output, BLOCK_SIZE_M=BLOCK_SIZE_M, BLOCK_SIZE_N=BLOCK_SIZE_N, BLOCK_SIZE_K=BLOCK_SIZE_K):
    """A batch of matmuls on 3-D operands (the shape of tensors docs/source/build.rst:237-245 of the reference project
    names for a batched matmul): the matmul tiling with a leading batch dimension of tile size 1, squeezed out of the
    tiles so that the matmul application runs on each (batch, m-tile, n-tile) unchanged."""
    output_tiled = output.tile((1, BLOCK_SIZE_M, BLOCK_SIZE_N))
    output_tiled.dtype = output_tiled.dtype.squeeze(0)

    lhs_tiled = lhs.tile((1, BLOCK_SIZE_M, BLOCK_SIZE_K)).tile((1, 1, -1)).expand((-1, -1, output_tiled.shape[2]))
    lhs_tiled.dtype = lhs_tiled.dtype.squeeze((0, 1))
    lhs_tiled.dtype.dtype = lhs_tiled.dtype.dtype.squeeze(0)

    rhs_tiled = rhs.tile((1, BLOCK_SIZE_K, BLOCK_SIZE_N)).tile((1, -1, 1)).expand((-1, output_tiled.shape[1], -1))
    rhs_tiled.dtype = rhs_tiled.dtype.squeeze((0, 2))
    rhs_tiled.dtype.dtype = rhs_tiled.dtype.dtype.squeeze(0)

    return lhs_tiled, rhs_tiled, output_tiled


def make_bmm(**kwargs):
    return ninetoothed.make(bmm_arrangement, matmul_application, (Tensor(3), Tensor(3), Tensor(3)), **kwargs)


# ------------------------------------------------------------------- addmm
def addmm_arrangement(input, mat1, mat2, beta, alpha, output, BLOCK_SIZE_M=BLOCK_SIZE_M, BLOCK_SIZE_N=BLOCK_SIZE_N,
                      BLOCK_SIZE_K=BLOCK_SIZE_K):
    _, _, input_arranged = matmul_arrangement(mat1, mat2, input, BLOCK_SIZE_M, BLOCK_SIZE_N, BLOCK_SIZE_K)
    mat1_arranged, mat2_arranged, output_arranged = matmul_arrangement(
        mat1, mat2, output, BLOCK_SIZE_M, BLOCK_SIZE_N, BLOCK_SIZE_K
    )
    return input_arranged, mat1_arranged, mat2_arranged, beta, alpha, output_arranged


def addmm_application(input, mat1, mat2, beta, alpha, output):
    matmul_output = ntl.zeros(output.shape, dtype=ntl.float32)
    matmul_application(mat1, mat2, matmul_output)
    output = beta * input + alpha * matmul_output  # noqa: F841


def make_addmm(**kwargs):
    return ninetoothed.make(
        addmm_arrangement, addmm_application,
        (Tensor(2), Tensor(2), Tensor(2), Tensor(0), Tensor(0), Tensor(2)), **kwargs,
    )


# ----------------------------------------------------------------- softmax
def make_softmax():
    BLOCK_SIZE = Symbol("BLOCK_SIZE", constexpr=True)

    @ninetoothed.jit
    def softmax_kernel(
        input_row: Tensor(2, other=float("-inf")).tile((1, BLOCK_SIZE)),
        output_row: Tensor(2).tile((1, BLOCK_SIZE)),
    ):
        row_minus_max = input_row - ntl.max(input_row)
        numerator = ntl.exp(row_minus_max)
        denominator = ntl.sum(numerator)
        output_row = numerator / denominator  # noqa: F841

    return softmax_kernel


def make_softmax_fp32_math():
    """fp16/bf16 storage: the row is widened before exp, as Triton's exp requires."""
    BLOCK_SIZE = Symbol("BLOCK_SIZE", constexpr=True)

    def arrangement(input, output, BLOCK_SIZE=BLOCK_SIZE):
        return input.tile((1, BLOCK_SIZE)), output.tile((1, BLOCK_SIZE))

    def application(input_row, output_row):
        loaded = input_row
        row = loaded.to(ntl.float32)
        row_minus_max = row - ntl.max(row)
        numerator = ntl.exp(row_minus_max)
        denominator = ntl.sum(numerator)
        output_row = numerator / denominator  # noqa: F841

    return ninetoothed.make(arrangement, application, (Tensor(2, other=float("-inf")), Tensor(2)))


# --------------------------------------------------------------- attention
ATTENTION_BLOCK_SIZE_M = block_size(lower_bound=64, upper_bound=128)
ATTENTION_BLOCK_SIZE_N = block_size(lower_bound=32, upper_bound=64)


def attention_arrangement(q, k, v, is_causal, o, BLOCK_SIZE_M=ATTENTION_BLOCK_SIZE_M,
                          BLOCK_SIZE_N=ATTENTION_BLOCK_SIZE_N):
    def arrange_q_or_o(input):
        arranged = input.tile((1, 1, BLOCK_SIZE_M, -1))
        arranged.dtype = arranged.dtype.squeeze((0, 1))
        return arranged

    def arrange_k_or_v(input):
        arranged = (
            input.tile((1, 1, BLOCK_SIZE_N, -1)).tile((1, 1, -1, -1)).expand((-1, -1, q_arranged.shape[-2], -1))
        )
        arranged.dtype = arranged.dtype.squeeze((0, 1, 3))
        arranged.dtype.dtype = arranged.dtype.dtype.squeeze((0, 1))
        return arranged

    q_arranged = arrange_q_or_o(q)
    return q_arranged, arrange_k_or_v(k), arrange_k_or_v(v), is_causal, arrange_q_or_o(o)


def attention_application(q, k, v, is_causal, o):
    q_loaded = (q * 1.44269504089).to(q.dtype)

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
    o = acc  # noqa: F841


def _attention_tensor():
    return Tensor(4, shape_options=(None, None, {"constexpr": True}, {"constexpr": True, "upper_bound": 128}))


def make_attention():
    tensors = (_attention_tensor(), _attention_tensor(), _attention_tensor(), Tensor(0, constexpr=True),
               _attention_tensor())
    return ninetoothed.make(attention_arrangement, attention_application, tensors)


def scaled_attention_arrangement(q, k, v, scale, is_causal, o):
    q_arranged, k_arranged, v_arranged, causal, o_arranged = attention_arrangement(q, k, v, is_causal, o)
    return q_arranged, k_arranged, v_arranged, scale, causal, o_arranged


def scaled_attention_application(q, k, v, scale, is_causal, o):
    q_loaded = (q * scale * 1.44269504089).to(q.dtype)

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
    o = acc  # noqa: F841


def make_scaled_attention():
    tensors = (_attention_tensor(), _attention_tensor(), _attention_tensor(), Tensor(0), Tensor(0, constexpr=True),
               _attention_tensor())
    return ninetoothed.make(scaled_attention_arrangement, scaled_attention_application, tensors)


# ------------------------------------------------------------------ conv2d
def conv2d_arrangement(input, filter, output, enable_padding=False, BLOCK_SIZE_M=BLOCK_SIZE_M,
                       BLOCK_SIZE_N=BLOCK_SIZE_N, BLOCK_SIZE_K=BLOCK_SIZE_K):
    if enable_padding:
        padding_h = Symbol("padding_h", constexpr=True)
        padding_w = Symbol("padding_w", constexpr=True)
        pad = ((0, 0), (0, 0), (padding_h, padding_h), (padding_w, padding_w))
        input_padded = input.pad(pad)
    else:
        input_padded = input

    input_tiled = input_padded.tile((1, *filter.shape[1:]), strides=(-1, -1, 1, 1))
    input_squeezed = input_tiled.squeeze(1)
    input_squeezed.dtype = input_squeezed.dtype.squeeze(0)
    input_raveled = input_squeezed.ravel()
    input_flattened = input_raveled.flatten(end_dim=3).flatten(start_dim=1)

    filter_flattened = filter.flatten(start_dim=1)
    filter_permuted = filter_flattened.permute((1, 0))

    output_flattened = output.permute((0, 2, 3, 1)).flatten(end_dim=3)

    return functools.partial(
        matmul_arrangement, BLOCK_SIZE_M=BLOCK_SIZE_M, BLOCK_SIZE_N=BLOCK_SIZE_N, BLOCK_SIZE_K=BLOCK_SIZE_K
    )(input_flattened, filter_permuted, output_flattened)


def conv2d_premake(n=None, c=None, h=None, w=None, k=None, r=None, s=None, dtype=None, block_size_m=64,
                   block_size_n=64, block_size_k=64):
    """The premake of the reference's conv2d test (tests/test_conv2d.py:51-87): arrangement with the
    given block sizes, the matmul application, tensors with the given (possibly unknown) sizes."""
    arrangement = functools.partial(conv2d_arrangement, BLOCK_SIZE_M=block_size_m, BLOCK_SIZE_N=block_size_n,
                                    BLOCK_SIZE_K=block_size_k)
    p = h - r + 1 if h is not None and r is not None else None
    q = w - s + 1 if w is not None and s is not None else None
    tensors = (Tensor(shape=(n, c, h, w), dtype=dtype), Tensor(shape=(k, c, r, s), dtype=dtype),
               Tensor(shape=(n, k, p, q), dtype=dtype))
    return arrangement, matmul_application, tensors


def make_conv2d(enable_padding=True):
    return ninetoothed.make(
        functools.partial(conv2d_arrangement, enable_padding=enable_padding),
        matmul_application,
        (Tensor(4), Tensor(4, shape_options={"constexpr": True}), Tensor(4)),
        max_num_configs=50,
    )


# -------------------------------------------------------------- max_pool2d
def max_pool2d_arrangement(input, output, ceil_mode=False):
    BLOCK_SIZE = Symbol("BLOCK_SIZE", meta=True)

    WINDOW_HEIGHT = Symbol("WINDOW_HEIGHT", constexpr=True, upper_bound=16)
    WINDOW_WIDTH = Symbol("WINDOW_WIDTH", constexpr=True, upper_bound=16)

    input_arranged = input.tile((1, 1, WINDOW_HEIGHT, WINDOW_WIDTH), floor_mode=not ceil_mode)
    input_arranged = input_arranged.ravel()
    input_arranged = input_arranged.flatten(end_dim=4).flatten(start_dim=1)
    input_arranged = input_arranged.tile((BLOCK_SIZE, -1))

    output_arranged = output.tile((1, 1, 1, 1))
    output_arranged = output_arranged.ravel()
    output_arranged = output_arranged.flatten(end_dim=4).flatten(start_dim=1)
    output_arranged = output_arranged.tile((BLOCK_SIZE, -1))
    output_arranged.dtype = output_arranged.dtype.squeeze(1)

    return input_arranged, output_arranged


def max_pool2d_application(input, output):
    output = ntl.max(input, axis=1)  # noqa: F841


@functools.lru_cache(maxsize=None)
def make_max_pool2d(ceil_mode=False):
    return ninetoothed.make(functools.partial(max_pool2d_arrangement, ceil_mode=ceil_mode), max_pool2d_application,
                            (Tensor(4, other=float("-inf")), Tensor(4)))
