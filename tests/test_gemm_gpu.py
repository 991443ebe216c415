"""matmul / addmm on the GPU, through the C ABI, against the oracle and the golden vectors.

Mirrors the reference's tests/test_matmul.py and tests/test_addmm.py (512^3 fp16 vs
torch) and adds ragged shapes, transposed views and the epilogue's rounding rule.
Tolerance: rtol 1e-2 / atol 1e-2 on fp16 outputs whose magnitude is ~sqrt(K); the
epilogue rounding rule is additionally checked bit for bit on exact inputs.
"""

import numpy as np
import pytest
import torch

from oracle import inputs as oi
from oracle import kernels as ok

from conftest import load_golden
from gpu_util import assert_close, assert_device_healthy, dev, host

pytestmark = pytest.mark.gpu


def run_matmul(a, b):
    from ninetoothed_b200 import _capi

    ad, bd = dev(a), dev(b)
    out = torch.empty((a.shape[0], b.shape[1]), dtype=ad.dtype, device="cuda")
    _capi.matmul(ad, bd, out)
    torch.cuda.synchronize()
    return host(out)


def run_addmm(c, a, b, beta, alpha):
    from ninetoothed_b200 import _capi

    cd, ad, bd = dev(c), dev(a), dev(b)
    out = torch.empty((a.shape[0], b.shape[1]), dtype=ad.dtype, device="cuda")
    _capi.addmm(cd, ad, bd, beta, alpha, out)
    torch.cuda.synchronize()
    return host(out)


def close_in_ulps(actual, expected, k):
    """Much tighter than the 1e-2 bar.  The tensor core adds the K products in
    another order than the oracle, which moves the fp32 accumulator by about
    1e-6 * k in absolute terms before the single fp16 rounding: allow that plus one
    fp16 unit in the last place, and require almost all elements bit-identical."""
    a = actual.astype(np.float32)
    e = expected.astype(np.float32)
    ulp = np.spacing(np.abs(e).astype(np.float16)).astype(np.float32)
    assert (np.abs(a - e) <= ulp + 2e-6 * k).all()
    assert (a == e).mean() > 0.97


@pytest.mark.parametrize("case", sorted(load_golden("matmul")))
def test_matmul_golden(case):
    g = load_golden("matmul")[case]
    m, n, k = (int(v) for v in g["shape"])
    a, b = oi.matmul_inputs(m, n, k, int(g["seed"]))
    out = run_matmul(a, b)
    assert_close(out, g["out"])
    close_in_ulps(out, g["out"], k)
    assert_device_healthy()


@pytest.mark.parametrize("case", sorted(load_golden("addmm")))
def test_addmm_golden(case):
    g = load_golden("addmm")[case]
    m, n, k = (int(v) for v in g["shape"])
    c, a, b = oi.addmm_inputs(m, n, k, int(g["seed"]))
    out = run_addmm(c, a, b, float(g["beta"]), float(g["alpha"]))
    assert_close(out, g["out"])
    # two extra roundings in the epilogue: allow 2 fp16 ulps
    ulp = np.spacing(np.abs(g["out"]).astype(np.float16)).astype(np.float32)
    assert (np.abs(out.astype(np.float32) - g["out"].astype(np.float32)) <= 2 * ulp + 1e-3).all()
    assert_device_healthy()


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (384, 768, 1024),
                                     (1000, 520, 264), (8, 8, 8), (130, 264, 72), (2048, 2048, 2048),
                                     # enough 256 x 256 tiles to switch to the CTA-pair kernel
                                     (2304, 2304, 512), (2500, 2312, 264),
                                     # shapes for which the launcher picks 128- and 64-column tiles, ragged in N
                                     (1024, 2040, 320), (1000, 1000, 192)])
def test_matmul_shapes(m, n, k):
    a, b = oi.matmul_inputs(m, n, k, 20 + m)
    out = run_matmul(a, b)
    expected = ok.matmul(a, b, np.float16, 128, 256, 64)
    assert_close(out, expected)
    close_in_ulps(out, expected, k)
    assert_device_healthy()


def test_matmul_integer_inputs_are_exact():
    """Small integers make every product and partial sum exact in fp32 and fp16."""
    rng = np.random.default_rng(3)
    a = rng.integers(-3, 4, size=(256, 320)).astype(np.float16)
    b = rng.integers(-3, 4, size=(320, 512)).astype(np.float16)
    out = run_matmul(a, b)
    expected = (a.astype(np.float32) @ b.astype(np.float32)).astype(np.float16)
    assert np.array_equal(out, expected)


def test_addmm_epilogue_rounds_in_storage_type():
    """beta*input + alpha*fp16(A.B) with every operation rounded to fp16: bit exact
    on integer-valued A, B (exact product) against the oracle's rule."""
    rng = np.random.default_rng(4)
    a = rng.integers(-3, 4, size=(128, 192)).astype(np.float16)
    b = rng.integers(-3, 4, size=(192, 256)).astype(np.float16)
    c = oi.normal(5, (128, 256))
    out = run_addmm(c, a, b, -1.3, 0.7)
    expected = ok.addmm(c, a, b, -1.3, 0.7, np.float16, 128, 256, 64)
    assert np.array_equal(out, expected)


def test_transposed_rhs_and_row_padded_views():
    from ninetoothed_b200 import _capi

    a, b = oi.matmul_inputs(256, 384, 320, 31)
    expected = ok.matmul(a, b, np.float16, 128, 256, 64)
    ad = dev(a)
    bt = dev(np.ascontiguousarray(b.T)).t()  # [K, N] view with unit stride along K
    out = torch.empty(256, 384, dtype=torch.float16, device="cuda")
    _capi.matmul(ad, bt, out)
    close_in_ulps(host(out), expected, 320)
    # output and lhs as column slices of wider buffers
    wide_a = torch.zeros(256, 512, dtype=torch.float16, device="cuda")
    wide_a[:, :320] = ad
    wide_out = torch.zeros(256, 640, dtype=torch.float16, device="cuda")
    _capi.matmul(wide_a[:, :320], dev(b), wide_out[:, 128:512])
    close_in_ulps(host(wide_out[:, 128:512]), expected, 320)
    assert float(wide_out[:, :128].abs().sum()) == 0 and float(wide_out[:, 512:].abs().sum()) == 0
    # an lhs no TMA descriptor can address (unit stride along M) takes the plain kernel
    at = dev(np.ascontiguousarray(a.T)).t()
    _capi.matmul(at, dev(b), out)
    close_in_ulps(host(out), expected, 320)
    assert_device_healthy()


@pytest.mark.parametrize("m, n, k", [
    (512, 512, 4096),     # 8 tiles for 148 SMs: every tile is summed from many partial accumulators
    (1024, 1024, 8192),   # 32 tiles, four or five partials each
    (700, 520, 4104),     # ragged in M, N and K
    (256, 264, 16384),    # two tiles, the second one 8 columns wide
    (1024, 1024, 1024),   # too short a reduction to split: the ordinary launch
])
def test_split_along_k_is_exact_and_repeatable(m, n, k):
    """A problem with too few tiles for the device is cut along K: every CTA accumulates a run of
    k-blocks, and a second kernel adds a tile's partial accumulators up in a fixed order.
    Integer-valued operands make every partial sum exact, so the result must equal the fp32 product
    bit for bit; on N(0,1) operands two runs must agree bit for bit."""
    from ninetoothed_b200 import _capi

    rng = np.random.default_rng(m + k)
    a = rng.integers(-2, 3, size=(m, k)).astype(np.float16)
    b = rng.integers(-2, 3, size=(k, n)).astype(np.float16)
    expected = (a.astype(np.float32) @ b.astype(np.float32)).astype(np.float16)
    assert np.array_equal(run_matmul(a, b), expected)
    c = rng.integers(-8, 9, size=(m, n)).astype(np.float16)
    assert np.array_equal(run_addmm(c, a, b, 1.0, 1.0), (expected.astype(np.float32) + c.astype(np.float32)).astype(np.float16))
    a, b = oi.matmul_inputs(m, n, k, 77)
    ad, bd = dev(a), dev(b)
    first = torch.empty((m, n), dtype=torch.float16, device="cuda")
    again = torch.empty_like(first)
    _capi.matmul(ad, bd, first)
    for _ in range(3):
        _capi.matmul(ad, bd, again)
        assert torch.equal(first, again)
    reference = (ad.float() @ bd.float()).half()
    assert_close(host(first), host(reference))
    assert_device_healthy()


@pytest.mark.parametrize("m, n, k", [(1024, 2040, 320), (1000, 1000, 192)])
def test_narrow_tiles_addmm_and_transposed_rhs(m, n, k):
    """128- and 64-column tiles: the addmm epilogue, and rhs as a transposed view (K-major B)."""
    from ninetoothed_b200 import _capi

    c, a, b = oi.addmm_inputs(m, n, k, 50 + k)
    expected = ok.addmm(c, a, b, 0.75, -1.5, np.float16, 128, 256, 64)
    assert_close(run_addmm(c, a, b, 0.75, -1.5), expected)
    bt = dev(np.ascontiguousarray(b.T)).t()
    out = torch.empty(m, n, dtype=torch.float16, device="cuda")
    _capi.matmul(dev(a), bt, out)
    close_in_ulps(host(out), ok.matmul(a, b, np.float16, 128, 256, 64), k)
    assert_device_healthy()


def test_addmm_on_the_cta_pair_kernel():
    """Large enough for 256 x 256 tiles; ragged in M and N; non-unit scalars."""
    m, n, k = 2400, 2360, 320
    c, a, b = oi.addmm_inputs(m, n, k, 33)
    out = run_addmm(c, a, b, 0.75, -1.5)
    expected = ok.addmm(c, a, b, 0.75, -1.5, np.float16, 256, 256, 64)
    assert_close(out, expected)
    # the summation order moves fp16(A.B) by one unit in the last place on a few elements; all others are bit-identical
    assert (out == expected).mean() > 0.99
    assert_device_healthy()


def test_bf16():
    from ninetoothed_b200 import _capi

    a, b = oi.matmul_inputs(256, 256, 512, 41, dtype=np.float32)
    ad, bd = torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16()
    out = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    _capi.matmul(ad, bd, out)
    expected = host(ad.float()) @ host(bd.float())
    assert_close(host(out.float()), expected, rtol=1e-2, atol=0.15)


def test_addmm_8192_linearity():
    """Full benchmark size: out(alpha=1,beta=1) - out(alpha=1,beta=0) == input, up to
    the fp16 roundings, and a sampled block against the oracle."""
    from ninetoothed_b200 import _capi

    g = torch.Generator(device="cuda").manual_seed(1)
    n = 8192
    c = torch.randn(n, n, generator=g, device="cuda", dtype=torch.float32).half()
    a = torch.randn(n, n, generator=g, device="cuda", dtype=torch.float32).half()
    b = torch.randn(n, n, generator=g, device="cuda", dtype=torch.float32).half()
    out = torch.empty(n, n, dtype=torch.float16, device="cuda")
    prod = torch.empty(n, n, dtype=torch.float16, device="cuda")
    _capi.addmm(c, a, b, 1.0, 1.0, out)
    _capi.matmul(a, b, prod)
    assert torch.equal(out, c + prod)  # fp16(c + fp16(ab)): one exact rule, bit for bit
    rows = slice(4096 - 64, 4096 + 64)
    cols = slice(8192 - 256, 8192)
    expected = ok.matmul(host(a[rows]), host(b[:, cols]), np.float16, 128, 256, 64)
    assert_close(host(prod[rows, cols]), expected)
    assert_device_healthy()


def test_rejects_bad_arguments():
    from ninetoothed_b200 import _capi

    a = torch.zeros(16, 32, dtype=torch.float16, device="cuda")
    b = torch.zeros(16, 32, dtype=torch.float16, device="cuda")
    out = torch.zeros(16, 32, dtype=torch.float16, device="cuda")
    with pytest.raises(_capi.KernelLaunchError):
        _capi.matmul(a, b, out)
    with pytest.raises(_capi.KernelLaunchError):
        _capi.matmul(a.float(), b.float().t(), torch.zeros(16, 16, device="cuda"))


# ------------------------------------------------------------------ 8-bit e5m2 operands
def run_matmul_e5m2(a8, b8_view):
    """a8: uint8 [M, K]; b8_view: uint8 [K, N] view (any strides); fp16 output."""
    from examples import definitions as kd

    lhs = torch.from_numpy(np.ascontiguousarray(a8)).cuda().view(torch.float8_e5m2)
    base = torch.from_numpy(np.ascontiguousarray(b8_view.base if b8_view.base is not None else b8_view)).cuda()
    rhs = (base.T if b8_view.base is not None else base).view(torch.float8_e5m2)
    assert tuple(rhs.shape) == tuple(b8_view.shape)
    out = torch.empty((a8.shape[0], b8_view.shape[1]), dtype=torch.float16, device="cuda")
    kd.make_matmul()(lhs, rhs, out)
    torch.cuda.synchronize()
    return host(out)


@pytest.mark.parametrize("case", sorted(load_golden("matmul_e5m2")))
def test_matmul_e5m2_golden(case):
    g = load_golden("matmul_e5m2")[case]
    m, n, k = (int(v) for v in g["shape"])
    a8, bt8 = oi.matmul_e5m2_inputs(m, n, k, int(g["seed"]))
    out = run_matmul_e5m2(a8, bt8.T)
    assert_close(out, g["out"])
    assert_device_healthy()


@pytest.mark.parametrize("m, n, k", [(512, 512, 512), (300, 200, 160), (2304, 2304, 256), (130, 70, 48)])
def test_matmul_e5m2_shapes(m, n, k):
    """tests/test_matmul.py:72-90 of the reference (512^3, atol 0.125 against torch on the decoded operands),
    a ragged shape, one that takes the CTA-pair kernel, and a K whose rows are 16-byte addressable but
    not a multiple of the 128-element stage."""
    a8, bt8 = oi.matmul_e5m2_inputs(m, n, k, 60 + k)
    out = run_matmul_e5m2(a8, bt8.T)
    a16, b16 = oi.e5m2_to_fp16(a8), oi.e5m2_to_fp16(bt8).T
    expected = torch.matmul(dev(a16).float(), dev(np.ascontiguousarray(b16)).float())
    assert np.abs(out.astype(np.float32) - host(expected)).max() <= 0.125
    close_in_ulps(out, ok.matmul(a16, b16, np.float16, 128, 256, 64), k)
    assert_device_healthy()


def test_matmul_e5m2_row_major_rhs_takes_the_plain_kernel():
    a8, bt8 = oi.matmul_e5m2_inputs(96, 80, 72, 61)
    b8 = np.ascontiguousarray(bt8.T)  # [K, N] with unit stride along N: no tensor-core path for 8-bit operands
    out = run_matmul_e5m2(a8, b8)
    close_in_ulps(out, ok.matmul(oi.e5m2_to_fp16(a8), oi.e5m2_to_fp16(b8), np.float16, 128, 256, 64), 72)
    assert_device_healthy()


# ------------------------------------------------------------------ bmm: a batch of matmuls
def run_bmm(a, b, out=None):
    from examples import definitions as kd

    ad, bd = (t if isinstance(t, torch.Tensor) else dev(t) for t in (a, b))
    if out is None:
        out = torch.empty((ad.shape[0], ad.shape[1], bd.shape[2]), dtype=ad.dtype, device="cuda")
    kd.make_bmm()(ad, bd, out)
    torch.cuda.synchronize()
    return host(out)


@pytest.mark.parametrize("case", ["square", "ragged"])
def test_bmm_golden(case):
    g = load_golden("bmm")[case]
    batch, m, n, k = (int(v) for v in g["shape"])
    seed = int(g["seed"])
    a, b = ok.normal(seed, (batch, m, k), np.float16), ok.normal(seed + 1000, (batch, k, n), np.float16)
    out = run_bmm(a, b)
    assert_close(out, g["out"])
    close_in_ulps(out, g["out"], k)
    assert_device_healthy()


@pytest.mark.parametrize("batch, m, n, k", [(1, 128, 256, 64), (5, 300, 136, 200), (16, 64, 64, 64), (3, 257, 520, 72),
                                            (2, 1024, 1024, 512), (7, 8, 8, 8)])
def test_bmm_shapes(batch, m, n, k):
    """One launch for all problems (3-D tensor maps; rows of a tile past M must read zeros, not the next problem)."""
    a, b = ok.normal(40 + batch, (batch, m, k), np.float16), ok.normal(41 + batch, (batch, k, n), np.float16)
    out = run_bmm(a, b)
    expected = ok.bmm(a, b)
    assert_close(out, expected)
    close_in_ulps(out, expected, k)
    assert_device_healthy()


def test_bmm_strided_operands_bf16_and_empty():
    from ninetoothed_b200 import _capi

    a, b = ok.normal(50, (4, 96, 80), np.float16), ok.normal(51, (4, 80, 72), np.float16)
    expected = ok.bmm(a, b)
    # rhs as a transposed view (unit stride along K): one matmul launch per problem
    bt = dev(np.ascontiguousarray(b.transpose(0, 2, 1))).transpose(1, 2)
    assert_close(run_bmm(dev(a), bt), expected)
    # output rows inside a wider buffer, batch stride not the dense one
    wide = torch.zeros(4, 96, 128, dtype=torch.float16, device="cuda")
    run_bmm(dev(a), dev(b), wide[:, :, 8:80])
    assert_close(host(wide[:, :, 8:80]), expected)
    assert float(wide[:, :, :8].abs().max()) == 0 and float(wide[:, :, 80:].abs().max()) == 0
    # K not a multiple of 8: rows that TMA cannot address
    a2, b2 = ok.normal(52, (2, 40, 30), np.float16), ok.normal(53, (2, 30, 24), np.float16)
    assert_close(run_bmm(a2, b2), ok.bmm(a2, b2))
    # bf16
    ab, bb = dev(a).bfloat16(), dev(b).bfloat16()
    out = torch.empty(4, 96, 72, dtype=torch.bfloat16, device="cuda")
    _capi.bmm(ab, bb, out)
    ref = torch.bmm(ab.float(), bb.float())
    assert_close(out.float().cpu().numpy(), ref.cpu().numpy(), rtol=2e-2, atol=2e-2)
    # an empty batch launches nothing
    _capi.bmm(torch.empty(0, 8, 8, dtype=torch.float16, device="cuda"), torch.empty(0, 8, 8, dtype=torch.float16, device="cuda"),
              torch.empty(0, 8, 8, dtype=torch.float16, device="cuda"))
    with pytest.raises(_capi.KernelLaunchError):
        _capi.bmm(dev(a), dev(b[:3]), torch.empty(4, 96, 72, dtype=torch.float16, device="cuda"))
    assert_device_healthy()


@pytest.mark.parametrize(
    "m, n, k, mode, transposed_rhs, dtype",
    [
        (8192, 1024, 320, None, False, torch.float16),     # 128 tiles on the device's CTA pairs: the planner mixes by itself
        (4096, 4096, 192, None, False, torch.float16),     # 256 tiles
        (8000, 1000, 320, "force", False, torch.float16),  # ragged rows and a ragged last narrow tile
        (8192, 2048, 128, "force", False, torch.bfloat16), # two swaps per tile-row
        (8192, 1024, 256, "force", True, torch.float16),   # rhs as a transposed view (K-major tiles)
        (8192, 1280, 192, "force", False, torch.float16),  # wide tiles after the swaps: [256, 256, 192 x 4]
    ],
)
def test_mixed_tile_widths_do_not_change_a_bit(monkeypatch, m, n, k, mode, transposed_rhs, dtype):
    """Launches whose last wave of CTA pairs would be mostly idle trade 256-column tiles for 192-column ones.
    The reduction order inside a tile does not depend on its width, so the output must equal, bit for bit, the
    one computed with the trade switched off; and it must be right."""
    from ninetoothed_b200 import _capi

    gen = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=gen, device="cuda").to(dtype)
    b = torch.randn(n, k, generator=gen, device="cuda").to(dtype).T if transposed_rhs else \
        torch.randn(k, n, generator=gen, device="cuda").to(dtype)
    c = torch.randn(m, n, generator=gen, device="cuda").to(dtype)

    def both():
        out_mm = torch.empty(m, n, dtype=dtype, device="cuda")
        out_add = torch.empty(m, n, dtype=dtype, device="cuda")
        _capi.matmul(a, b, out_mm)
        _capi.addmm(c, a, b, 0.5, 2.0, out_add)
        torch.cuda.synchronize()
        return out_mm, out_add

    monkeypatch.setenv("NINETOOTHED_B200_GEMM_MIXED", "0")
    _capi.mixed_width_launches(reset=True)
    plain_mm, plain_add = both()
    assert _capi.mixed_width_launches() == 0
    if mode is None:
        monkeypatch.delenv("NINETOOTHED_B200_GEMM_MIXED")
    else:
        monkeypatch.setenv("NINETOOTHED_B200_GEMM_MIXED", mode)
    mixed_mm, mixed_add = both()
    assert _capi.mixed_width_launches(reset=True) == 2, "the launches did not take the mixed-width path"
    assert torch.equal(mixed_mm, plain_mm)
    assert torch.equal(mixed_add, plain_add)
    expected = a.float() @ b.float()
    assert_close(host(mixed_mm.float()), host(expected.to(dtype).float()))
    assert_device_healthy()
