"""Fused attention on the GPU, through the C ABI, against the oracle and the golden vectors.

Mirrors the reference's tests/test_attention.py (B=2, H=4, S in {1024, 1}, D=64,
causal and not, fp16 rtol=atol=0.01 and fp32 0.025 against
scaled_dot_product_attention with scale=1) and adds D=128 with the 1/sqrt(D) scale,
ragged sequence lengths and strided views.  Tolerance: rtol 1e-2 / atol 1e-2.
"""

import numpy as np
import pytest
import torch

from oracle import inputs as oi
from oracle import kernels as ok

from conftest import load_golden
from gpu_util import assert_close, assert_device_healthy, dev, host

pytestmark = pytest.mark.gpu


def run(q, k, v, is_causal, scale=None):
    from ninetoothed_b200 import _capi

    qd, kd, vd = dev(q), dev(k), dev(v)
    o = torch.empty_like(qd)
    _capi.attention(qd, kd, vd, is_causal, o, scale=scale)
    torch.cuda.synchronize()
    return host(o)


@pytest.mark.parametrize("case", sorted(load_golden("attention")))
def test_golden(case):
    g = load_golden("attention")[case]
    shape = tuple(int(v) for v in g["shape"])
    q, k, v = oi.attention_inputs(shape, int(g["seed"]))
    scale = float(g["scale"])
    out = run(q, k, v, bool(g["is_causal"]), None if scale < 0 else scale)
    assert_close(out, g["out"])
    assert_device_healthy()


@pytest.mark.parametrize("is_causal", [False, True])
@pytest.mark.parametrize("seq_len", [1024, 1])
def test_reference_test_shapes_fp16(seq_len, is_causal):
    """tests/test_attention.py:99-117 of the reference, fp16 leg, against torch with scale=1."""
    shape = (2, 4, seq_len, 64)
    q, k, v = oi.attention_inputs(shape, 50 + seq_len)
    out = run(q, k, v, is_causal)
    expected = torch.nn.functional.scaled_dot_product_attention(
        dev(q).float(), dev(k).float(), dev(v).float(), is_causal=is_causal, scale=1)
    assert_close(out, host(expected), rtol=0.01, atol=0.01)
    assert_close(out, ok.attention(q, k, v, is_causal, 128, 128))


@pytest.mark.parametrize("is_causal", [False, True])
@pytest.mark.parametrize("seq_len", [79, 80, 81, 160, 255, 257, 336, 1000])
def test_sequence_lengths_around_the_tile_edges(seq_len, is_causal):
    """Key/value tiles are 80 rows, a CTA covers 256 query rows: lengths on, just under and just over
    both, with the softmax scale, against the oracle (64-key blocks there: only rounding order differs)."""
    shape = (1, 2, seq_len, 128)
    q, k, v = oi.attention_inputs(shape, 700 + seq_len)
    scale = ok.default_scale(128)
    out = run(q, k, v, is_causal, scale)
    assert_close(out, ok.attention(q, k, v, is_causal, 64, 64, scale=scale))
    assert_device_healthy()


def test_more_keys_than_queries_and_fewer():
    """q and k/v of different lengths (the kernel takes them; the reference's arrangement does too)."""
    from ninetoothed_b200 import _capi

    rng = np.random.default_rng(77)
    for s_q, s_kv in ((100, 333), (300, 90)):
        q = rng.standard_normal((1, 2, s_q, 64)).astype(np.float16)
        k = rng.standard_normal((1, 2, s_kv, 64)).astype(np.float16)
        v = rng.standard_normal((1, 2, s_kv, 64)).astype(np.float16)
        o = torch.empty(dev(q).shape, dtype=torch.float16, device="cuda")
        _capi.attention(dev(q), dev(k), dev(v), False, o, scale=0.125)
        torch.cuda.synchronize()
        expected = torch.nn.functional.scaled_dot_product_attention(
            dev(q).float(), dev(k).float(), dev(v).float(), scale=0.125)
        assert_close(host(o), host(expected))
    assert_device_healthy()


@pytest.mark.parametrize("is_causal", [False, True])
def test_reference_test_shape_fp32(is_causal):
    """fp32 leg of the reference test (rtol = atol = 0.025)."""
    from ninetoothed_b200 import _capi

    shape = (2, 4, 256, 64)
    q, k, v = (torch.from_numpy(x).cuda() for x in oi.attention_inputs(shape, 60, dtype=np.float32))
    o = torch.empty_like(q)
    _capi.attention(q, k, v, is_causal, o)
    expected = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=is_causal, scale=1)
    assert_close(host(o), host(expected), rtol=0.025, atol=0.025)


@pytest.mark.parametrize("shape, is_causal", [
    ((1, 1, 128, 128), False), ((1, 1, 128, 128), True), ((1, 2, 384, 128), True), ((2, 3, 200, 128), False),
    ((2, 3, 200, 128), True), ((1, 2, 130, 64), True), ((1, 1, 1000, 64), False), ((1, 1, 1, 128), True),
    ((2, 2, 2048, 128), True),
])
def test_scaled_shapes(shape, is_causal):
    q, k, v = oi.attention_inputs(shape, 70 + shape[2])
    scale = ok.default_scale(shape[3])
    out = run(q, k, v, is_causal, scale)
    assert_close(out, ok.attention(q, k, v, is_causal, 128, 128, scale=scale))
    assert_device_healthy()


def test_large_scores_trigger_rescaling():
    """Unscaled D=128 scores have a spread of ~16 in log2 units, so the running maximum
    moves by more than the lazy-rescale threshold several times per row."""
    shape = (1, 2, 1024, 128)
    q, k, v = oi.attention_inputs(shape, 81)
    for is_causal in (False, True):
        out = run(q, k, v, is_causal)
        assert_close(out, ok.attention(q, k, v, is_causal, 128, 128))


def test_plain_path_for_other_head_sizes_and_strides():
    from ninetoothed_b200 import _capi

    shape = (1, 2, 96, 80)  # head size 80: no tensor-core tiling here
    q, k, v = oi.attention_inputs(shape, 82)
    out = run(q, k, v, True, 0.1)
    assert_close(out, ok.attention(q, k, v, True, 64, 64, scale=0.1))
    # [B, S, H, D] storage viewed as [B, H, S, D]: strides (S*H*D, D, H*D, 1) go through TMA
    shape = (2, 4, 256, 64)
    q, k, v = oi.attention_inputs(shape, 83)
    views = [dev(x).permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3) for x in (q, k, v)]
    o = torch.empty(2, 256, 4, 64, dtype=torch.float16, device="cuda").permute(0, 2, 1, 3)
    _capi.attention(views[0], views[1], views[2], False, o)
    assert_close(host(o), ok.attention(q, k, v, False, 128, 128))
    assert_device_healthy()


def test_bf16():
    from ninetoothed_b200 import _capi

    shape = (1, 2, 512, 128)
    q, k, v = (torch.from_numpy(x).cuda().bfloat16() for x in oi.attention_inputs(shape, 84, dtype=np.float32))
    o = torch.empty_like(q)
    scale = ok.default_scale(128)
    _capi.attention(q, k, v, True, o, scale=scale)
    expected = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True,
                                                                scale=scale)
    assert_close(host(o.float()), host(expected), rtol=2e-2, atol=2e-2)


def test_full_size_properties():
    """B=4, H=32, S=4096, D=128: sampled heads against the oracle; with V = 1 every
    output is exactly 1 (softmax rows sum to 1), causal and not."""
    from ninetoothed_b200 import _capi

    g = torch.Generator(device="cuda").manual_seed(3)
    shape = (4, 32, 4096, 128)
    q, k, v = (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32).half() for _ in range(3))
    o = torch.empty_like(q)
    scale = ok.default_scale(128)
    for is_causal in (False, True):
        _capi.attention(q, k, v, is_causal, o, scale=scale)
        for b, h in ((0, 0), (3, 31)):
            sl = (slice(b, b + 1), slice(h, h + 1))
            expected = ok.attention(host(q[sl]), host(k[sl]), host(v[sl]), is_causal, 128, 128, scale=scale)
            assert_close(host(o[sl]), expected)
        ones = torch.ones_like(v)
        _capi.attention(q, k, ones, is_causal, o, scale=scale)
        assert (o.float() - 1).abs().max().item() < 2e-3
    assert_device_healthy()
