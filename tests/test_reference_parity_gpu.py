"""This library's kernels against the REFERENCE'S OWN kernels on the same device tensors.

The unmodified reference package (``baseline/_ref``, put there by
``baseline/install_reference.py``) compiles the definitions in ``examples/definitions.py``
to Triton kernels; this library's ``make`` handles get the same seeded device tensors at
the benchmark shapes, and the WHOLE outputs are compared at the bar the benchmark
states: rtol = atol = 1e-2 for fp16 results, softmax rows summing to 1 within 1e-3.
Block sizes are fixed (as the reference's README does), so nothing is tuned and each
reference kernel compiles in a second or two.  The module skips itself where the
reference is not installed.

torch's fp32 operators on the same tensors are a third opinion in the attention test,
which needs one: see ``test_attention_against_the_reference_and_fp32``.
"""

import pathlib
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from baseline import reference_runner as rr  # noqa: E402
from examples import definitions as kd  # noqa: E402

from gpu_util import assert_device_healthy  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not rr.available(), reason="the reference is not installed under baseline/_ref")]

RTOL = ATOL = 1e-2


def mismatches(actual, expected):
    """Elements outside |a - e| <= atol + rtol |e|, counted on the device over the whole tensor."""
    a, e = actual.float(), expected.float()
    return int(((a - e).abs() > ATOL + RTOL * e.abs()).sum().item()), float((a - e).abs().max().item())


def normal(shape, seed, scale=1.0):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    return (scale * torch.randn(shape, generator=generator, device="cuda", dtype=torch.float32)).half()


def test_readme_matmul_512():
    """Configuration 1 of the benchmark: the README matmul, 512^3, 64^3 blocks, seed 0."""
    generator = torch.Generator(device="cuda").manual_seed(0)
    lhs = torch.randn(512, 512, generator=generator, device="cuda").half()
    rhs = torch.randn(512, 512, generator=generator, device="cuda").half()
    ours, theirs = (torch.empty(512, 512, dtype=torch.float16, device="cuda") for _ in range(2))
    rr.matmul(blocks=(64, 64, 64), application="readme")(lhs, rhs, theirs)
    kd.ninetoothed.make(kd.matmul_arrangement, kd.readme_matmul_application, tuple(kd.Tensor(2) for _ in range(3)))(
        lhs, rhs, ours)
    bad, worst = mismatches(ours, theirs)
    assert bad == 0, (bad, worst)
    assert_device_healthy()


def test_addmm_8192():
    """Configuration 2: out = C + A.B at M = N = K = 8192, seed 1, compared over all 67M elements."""
    generator = torch.Generator(device="cuda").manual_seed(1)
    c, a, b = (torch.randn(8192, 8192, generator=generator, device="cuda", dtype=torch.float32).half()
               for _ in range(3))
    ours, theirs = (torch.empty(8192, 8192, dtype=torch.float16, device="cuda") for _ in range(2))
    rr.addmm(blocks=(128, 256, 64), num_warps=8, num_stages=3)(c, a, b, 1.0, 1.0, theirs)
    kd.make_addmm()(c, a, b, 1.0, 1.0, ours)
    bad, worst = mismatches(ours, theirs)
    assert bad == 0, (bad, worst)
    # both round the fp32 sum to fp16 once and add C in fp16: nearly every element is the same bits
    assert (ours == theirs).float().mean().item() > 0.99
    assert_device_healthy()


def test_softmax_65536x8192():
    """Configuration 3: rows of 8192 with entries 4 N(0,1), seed 2; rows sum to 1 within 1e-3."""
    x = normal((65536, 8192), 2, scale=4.0)
    ours, theirs = torch.empty_like(x), torch.empty_like(x)
    rr.softmax()(x, theirs, BLOCK_SIZE=8192)
    kd.make_softmax_fp32_math()(x, ours, BLOCK_SIZE=8192)
    bad, worst = mismatches(ours, theirs)
    assert bad == 0, (bad, worst)
    assert float((ours.float().sum(-1) - 1).abs().max().item()) < 1e-3
    assert_device_healthy()


def test_conv2d_64x256x56x56():
    """Configuration 5: 3x3 filters, 256 -> 256 channels, padding 1, seed 4."""
    generator = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(64, 256, 56, 56, generator=generator, device="cuda", dtype=torch.float32).half()
    w = (torch.randn(256, 256, 3, 3, generator=generator, device="cuda", dtype=torch.float32) / 2304 ** 0.5).half()
    ours, theirs = (torch.empty(64, 256, 56, 56, dtype=torch.float16, device="cuda") for _ in range(2))
    rr.conv2d(blocks=(128, 256, 64), num_warps=8, num_stages=3)(x, w, theirs, padding_h=1, padding_w=1)
    kd.make_conv2d()(x, w, ours, padding_h=1, padding_w=1)
    bad, worst = mismatches(ours, theirs)
    assert bad == 0, (bad, worst)
    assert_device_healthy()


@pytest.mark.parametrize("causal", [False, True])
def test_attention_against_the_reference_and_fp32(causal):
    """Configuration 4: B = 4, H = 32, S = 4096, D = 128, scale 1/sqrt(128), seed 3, whole output.

    The reference's attention body has no scale; the scaled form of examples/definitions.py folds a scalar
    into its pre-scale of q (one more 16-bit rounding of q, far inside the tolerance).  Both kernels are
    also held against torch's fp32 attention on every (batch, head) pair, eight pairs at a time."""
    import torch.nn.functional as F

    shape, scale = (4, 32, 4096, 128), 1.0 / 128 ** 0.5
    generator = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(shape, generator=generator, device="cuda", dtype=torch.float32).half() for _ in range(3))
    ours, theirs = torch.empty_like(q), torch.empty_like(q)
    rr.scaled_attention(blocks=(128, 32), num_warps=4, num_stages=3)(q, k, v, scale, causal, theirs)
    kd.make_scaled_attention()(q, k, v, scale, causal, ours)
    torch.cuda.synchronize()
    pairs = lambda t: t.reshape(128, 1, 4096, 128)  # noqa: E731
    ours_bad = theirs_bad = 0
    for first in range(0, 128, 8):
        rows = slice(first, first + 8)
        exact = F.scaled_dot_product_attention(pairs(q)[rows].float(), pairs(k)[rows].float(), pairs(v)[rows].float(),
                                               is_causal=causal, scale=scale)
        ours_bad += mismatches(pairs(ours)[rows], exact)[0]
        theirs_bad += mismatches(pairs(theirs)[rows], exact)[0]
        del exact
    bad, worst = mismatches(ours, theirs)
    assert ours_bad == 0, f"{ours_bad} elements of this library's output are off against fp32 attention"
    assert theirs_bad == 0, f"{theirs_bad} elements of the REFERENCE's output are off against fp32 attention"
    assert bad == 0, (bad, worst)
    assert_device_healthy()


def test_bmm_64x1024():
    """A "next" row: 64 independent 1024^3 matmuls on 3-D operands (the bench's bmm entry), whole output."""
    generator = torch.Generator(device="cuda").manual_seed(6)
    lhs, rhs = (torch.randn(64, 1024, 1024, generator=generator, device="cuda", dtype=torch.float32).half()
                for _ in range(2))
    ours, theirs = torch.empty_like(lhs), torch.empty_like(lhs)
    rr.bmm(blocks=(128, 128, 64), num_warps=8, num_stages=3)(lhs, rhs, theirs)
    kd.make_bmm()(lhs, rhs, ours)
    bad, worst = mismatches(ours, theirs)
    assert bad == 0, (bad, worst)
    assert (ours == theirs).float().mean().item() > 0.99
    assert_device_healthy()


@pytest.mark.parametrize("ceil_mode", [False, True])
def test_max_pool2d_64x256x112x112(ceil_mode):
    """A "next" row: 2 x 2 windows over [64, 256, 112, 112] (the bench's entry) and, ragged, over 111 x 109 pixels
    with floor and ceil tiling.  A maximum is exact: the outputs must be the same bits."""
    for height, width in ((112, 112), (111, 109)):
        x = normal((64, 256, height, width), 8)
        rows = -(-height // 2) if ceil_mode else height // 2
        cols = -(-width // 2) if ceil_mode else width // 2
        ours, theirs = (torch.empty(64, 256, rows, cols, dtype=torch.float16, device="cuda") for _ in range(2))
        rr.max_pool2d(ceil_mode)(x, theirs, WINDOW_HEIGHT=2, WINDOW_WIDTH=2)
        kd.make_max_pool2d(ceil_mode)(x, ours, WINDOW_HEIGHT=2, WINDOW_WIDTH=2)
        assert torch.equal(ours, theirs), (height, width, ceil_mode)
    assert_device_healthy()


def test_matmul_e5m2_4096():
    """A "next" row: 8-bit e5m2 operands, rhs as a transposed view, fp16 output (tests/test_matmul.py:60-90 of the
    reference project), 4096^3.  Products of e5m2 values are exact in fp32, so only the order of the sums differs."""
    if not hasattr(torch, "float8_e5m2"):
        pytest.skip("this torch has no float8_e5m2")
    generator = torch.Generator(device="cuda").manual_seed(9)
    lhs = torch.randn(4096, 4096, generator=generator, device="cuda").to(torch.float8_e5m2)
    rhs = torch.randn(4096, 4096, generator=generator, device="cuda").to(torch.float8_e5m2).T
    ours, theirs = (torch.empty(4096, 4096, dtype=torch.float16, device="cuda") for _ in range(2))
    rr.matmul(blocks=(128, 128, 64), num_warps=8, num_stages=3)(lhs, rhs, theirs)
    kd.make_matmul()(lhs, rhs, ours)
    bad, worst = mismatches(ours, theirs)
    assert bad == 0, (bad, worst)
    assert_device_healthy()


# ---------------------------------------------------------------------------------------------------
# The shapes, dtypes and value distributions of the reference's own tests (tests/test_addmm.py:55-75,
# test_softmax.py:28-40, test_attention.py:98-118, test_conv2d.py:112-133, test_max_pool2d.py:66-82 of the
# reference project), through both kernels.
# ---------------------------------------------------------------------------------------------------
def test_the_reference_tests_addmm_512():
    generator = torch.Generator(device="cuda").manual_seed(10)
    c, a, b = (torch.randn(512, 512, generator=generator, device="cuda").half() for _ in range(3))
    ours, theirs = torch.empty_like(c), torch.empty_like(c)
    for beta, alpha in ((0.37, 0.81), (1.0, 0.0), (0.0, 1.0)):
        rr.addmm(blocks=(64, 64, 64))(c, a, b, beta, alpha, theirs)
        kd.make_addmm()(c, a, b, beta, alpha, ours)
        bad, worst = mismatches(ours, theirs)
        assert bad == 0, (beta, alpha, bad, worst)
    assert_device_healthy()


def test_the_reference_tests_softmax_fp32_1823x781():
    generator = torch.Generator(device="cuda").manual_seed(11)
    x = torch.rand(1823, 781, generator=generator, device="cuda")
    ours, theirs = torch.empty_like(x), torch.empty_like(x)
    rr.plain_softmax()(x, theirs, BLOCK_SIZE=781)
    kd.make_softmax()(x, ours, BLOCK_SIZE=781)
    assert torch.allclose(ours, theirs, rtol=1e-5, atol=1e-7), float((ours - theirs).abs().max())
    assert torch.allclose(ours, torch.softmax(x, dim=-1))  # the reference test's own check
    assert_device_healthy()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype, tolerance", [(torch.float16, 0.01), (torch.float32, 0.025)])
@pytest.mark.parametrize("seq_len", [1024, 1])
def test_the_reference_tests_attention(seq_len, dtype, tolerance, causal):
    """[2, 4, S, 64], scale 1, fp16 and fp32 (the latter runs on this library's plain kernel)."""
    import warnings

    generator = torch.Generator(device="cuda").manual_seed(12)
    q, k, v = (torch.randn(2, 4, seq_len, 64, generator=generator, device="cuda").to(dtype) for _ in range(3))
    ours, theirs = torch.empty_like(q), torch.empty_like(q)
    rr.attention(blocks=(64, 32), num_warps=4, num_stages=2)(q, k, v, causal, theirs)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")  # fp32 attention announces that it runs on the plain kernel
        kd.make_attention()(q, k, v, causal, ours)
    a, e = ours.float(), theirs.float()
    assert int(((a - e).abs() > tolerance + tolerance * e.abs()).sum().item()) == 0, float((a - e).abs().max())
    assert_device_healthy()


@pytest.mark.parametrize("padding", [(0, 0), (1, 1), (0, 1), (2, 0)])
def test_the_reference_tests_conv2d(padding):
    """[4, 64, 16, 16] * [512, 64, 3, 3], uniform inputs, the reference test's four paddings and its 1e-3 bar."""
    generator = torch.Generator(device="cuda").manual_seed(13)
    x = torch.rand(4, 64, 16, 16, generator=generator, device="cuda").half()
    w = torch.rand(512, 64, 3, 3, generator=generator, device="cuda").half()
    p, q = 16 + 2 * padding[0] - 2, 16 + 2 * padding[1] - 2
    ours, theirs = (torch.empty(4, 512, p, q, dtype=torch.float16, device="cuda") for _ in range(2))
    rr.conv2d(blocks=(64, 64, 64), num_warps=4, num_stages=3)(x, w, theirs, padding_h=padding[0], padding_w=padding[1])
    kd.make_conv2d()(x, w, ours, padding_h=padding[0], padding_w=padding[1])
    assert torch.allclose(ours.float(), theirs.float(), rtol=1e-3, atol=1e-3), float((ours.float() - theirs.float()).abs().max())
    assert_device_healthy()


@pytest.mark.parametrize("ceil_mode", [False, True])
def test_the_reference_tests_max_pool2d(ceil_mode):
    """[32, 3, 64, 64], 3 x 3 windows."""
    x = normal((32, 3, 64, 64), 14)
    side = 22 if ceil_mode else 21
    ours, theirs = (torch.empty(32, 3, side, side, dtype=torch.float16, device="cuda") for _ in range(2))
    rr.max_pool2d(ceil_mode)(x, theirs, WINDOW_HEIGHT=3, WINDOW_WIDTH=3)
    kd.make_max_pool2d(ceil_mode)(x, ours, WINDOW_HEIGHT=3, WINDOW_WIDTH=3)
    assert torch.equal(ours, theirs)
    assert_device_healthy()


def test_bf16_through_both_kernels():
    """bf16 storage (the dtype of the reference's ahead-of-time tests, tests/test_aot.py:20 of the reference project):
    addmm 2048 x 1536 x 1024 and causal attention [2, 4, 1000, 128]; bf16 keeps 8 bits of mantissa, so the bar
    is 2e-2."""
    generator = torch.Generator(device="cuda").manual_seed(15)
    c = torch.randn(2048, 1536, generator=generator, device="cuda").bfloat16()
    a = torch.randn(2048, 1024, generator=generator, device="cuda").bfloat16()
    b = torch.randn(1024, 1536, generator=generator, device="cuda").bfloat16()
    ours, theirs = torch.empty_like(c), torch.empty_like(c)
    rr.addmm(blocks=(128, 128, 64), num_warps=8, num_stages=3)(c, a, b, 0.5, 1.5, theirs)
    kd.make_addmm()(c, a, b, 0.5, 1.5, ours)
    d, e = ours.float(), theirs.float()
    assert int(((d - e).abs() > 2e-2 + 2e-2 * e.abs()).sum().item()) == 0, float((d - e).abs().max())
    q, k, v = (torch.randn(2, 4, 1000, 128, generator=generator, device="cuda").bfloat16() for _ in range(3))
    ours, theirs = torch.empty_like(q), torch.empty_like(q)
    rr.attention(blocks=(64, 32), num_warps=4, num_stages=2)(q, k, v, True, theirs)
    kd.make_attention()(q, k, v, True, ours)
    d, e = ours.float(), theirs.float()
    assert int(((d - e).abs() > 2e-2 + 2e-2 * e.abs()).sum().item()) == 0, float((d - e).abs().max())
    assert_device_healthy()
