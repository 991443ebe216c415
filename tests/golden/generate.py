"""Regenerate the golden vectors in this directory from the reference itself.

Run by hand, in a container that has the reference checkout:

    python tests/golden/generate.py /path/to/reference [arrangements | max_pool2d | bmm]

(with a name: only that file, and for the first two the ones before it, is rewritten)

The reference is pure Python on top of Triton.  It is executed here on CPU by
Triton's interpreter (``TRITON_INTERPRET=1``) with block sizes fixed to ints so
no auto-tuning runs.  Two harness-side shims are installed, neither of which
edits the reference: a stub Triton driver (the reference asks the active driver
for register/shared-memory limits even when interpreting) and a fix-up for
string annotations in the interpreter's constexpr detection.

Inputs are NOT stored: they are re-drawn from ``oracle.kernels.normal`` with the
seeds recorded in each file, and a checksum of the inputs is stored to detect a
drifting generator.  Outputs of the reference kernels are stored bit for bit.
"""

import functools
import os
import pathlib
import sys
import time

os.environ["TRITON_INTERPRET"] = "1"

HERE = pathlib.Path(__file__).resolve().parent
REPO = HERE.parent.parent
if len(sys.argv) < 2:
    raise SystemExit(__doc__)
REFERENCE = pathlib.Path(sys.argv[1])
sys.path[:0] = [str(REPO), str(REFERENCE / "src"), str(REFERENCE)]

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402


class _Utils:
    def get_device_properties(self, device):
        return {"max_shared_mem": 232448, "max_num_regs": 65536, "multiprocessor_count": 148, "warpSize": 32}


class _StubDriver:
    utils = _Utils()

    def get_current_device(self):
        return 0

    def get_current_target(self):
        from triton.backends.compiler import GPUTarget

        return GPUTarget("cuda", 100, 32)

    def get_benchmarker(self):
        return lambda fn, quantiles=None, **kw: (fn(), [1.0, 1.0, 1.0])[1]

    def get_device_interface(self):
        return torch.cuda

    def get_active_torch_device(self):
        return torch.device("cpu")


try:
    triton.runtime.driver.active.get_current_device()
except Exception:
    triton.runtime.driver.set_active(_StubDriver())

import triton.runtime.jit as _jit  # noqa: E402

_normalize_ty = _jit._normalize_ty


def _normalize_ty_with_strings(ty):
    if isinstance(ty, str) and ty.strip().endswith(".constexpr"):
        return "constexpr"
    return _normalize_ty(ty)


_jit._normalize_ty = _normalize_ty_with_strings

import ninetoothed  # noqa: E402
import ninetoothed.language as ntl  # noqa: E402
import tests.test_addmm as ref_addmm  # noqa: E402
import tests.test_attention as ref_attention  # noqa: E402
import tests.test_conv2d as ref_conv2d  # noqa: E402
import tests.test_matmul as ref_matmul  # noqa: E402
import tests.test_max_pool2d as ref_max_pool2d  # noqa: E402
import tests.test_softmax as ref_softmax  # noqa: E402
from ninetoothed import Symbol, Tensor  # noqa: E402

from oracle import inputs as oi  # noqa: E402
from oracle import kernels as ok  # noqa: E402
from oracle.inputs import checksum  # noqa: E402


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def run_matmul(m, n, k, seed, blocks):
    a, b = oi.matmul_inputs(m, n, k, seed)
    out = torch.empty((m, n), dtype=torch.float16)
    kernel = ninetoothed.make(
        functools.partial(ref_matmul.arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1], BLOCK_SIZE_K=blocks[2]),
        ref_matmul.application,
        (Tensor(2), Tensor(2), Tensor(2)),
    )
    kernel(t(a), t(b), out)
    return dict(out=out.numpy(), inputs=checksum(a, b), seed=seed, shape=(m, n, k), blocks=blocks)


def run_matmul_e5m2(m, n, k, seed, blocks):
    """tests/test_matmul.py:60-90: e5m2 operands (rhs as a transposed view), fp16 output."""
    a8, bt8 = oi.matmul_e5m2_inputs(m, n, k, seed)
    a16, b16 = oi.matmul_inputs(m, n, k, seed)
    lhs = t(a16).to(torch.float8_e5m2)
    rhs = t(b16).T.contiguous().T.to(torch.float8_e5m2)  # [K, N] with unit stride along K
    # the numpy rounding used by the oracle's inputs is torch's
    assert np.array_equal(lhs.view(torch.uint8).numpy(), a8)
    assert np.array_equal(rhs.T.contiguous().view(torch.uint8).numpy(), bt8)
    assert rhs.stride() == (1, k)
    out = torch.empty((m, n), dtype=torch.float16)
    kernel = ninetoothed.make(
        functools.partial(ref_matmul.arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1], BLOCK_SIZE_K=blocks[2]),
        ref_matmul.application,
        (Tensor(2), Tensor(2), Tensor(2)),
    )
    kernel(lhs, rhs, out)
    return dict(out=out.numpy(), inputs=checksum(a8, bt8), seed=seed, shape=(m, n, k), blocks=blocks)


def run_addmm(m, n, k, seed, blocks, beta, alpha):
    c, a, b = oi.addmm_inputs(m, n, k, seed)
    out = torch.empty((m, n), dtype=torch.float16)
    kernel = ninetoothed.make(
        functools.partial(ref_addmm.arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1], BLOCK_SIZE_K=blocks[2]),
        ref_addmm.application,
        (Tensor(2), Tensor(2), Tensor(2), Tensor(0), Tensor(0), Tensor(2)),
    )
    kernel(t(c), t(a), t(b), beta, alpha, out)
    return dict(out=out.numpy(), inputs=checksum(c, a, b), seed=seed, shape=(m, n, k), blocks=blocks,
                beta=beta, alpha=alpha)


def run_softmax_fp32(rows, cols, seed):
    x = oi.softmax_inputs(rows, cols, seed, dtype=np.float32)
    out = ref_softmax.softmax(t(x))
    return dict(out=out.numpy(), inputs=checksum(x), seed=seed, shape=(rows, cols))


def run_softmax_fp16(rows, cols, seed, scale):
    """fp16 storage with fp32 math: the reference's definition plus a widening
    cast, because Triton's exp takes fp32/fp64 only."""
    block = Symbol("BLOCK_SIZE", constexpr=True)

    def arrangement(x, y, BLOCK_SIZE=block):
        return x.tile((1, BLOCK_SIZE)), y.tile((1, BLOCK_SIZE))

    def application(input_row, output_row):
        loaded = input_row
        row = loaded.to(ntl.float32)
        row_minus_max = row - ntl.max(row)
        numerator = ntl.exp(row_minus_max)
        denominator = ntl.sum(numerator)
        output_row = numerator / denominator  # noqa: F841

    x = oi.softmax_inputs(rows, cols, seed, scale=scale)
    out = torch.empty((rows, cols), dtype=torch.float16)
    kernel = ninetoothed.make(arrangement, application, (Tensor(2, other=float("-inf")), Tensor(2)))
    kernel(t(x), out, BLOCK_SIZE=cols)
    return dict(out=out.numpy(), inputs=checksum(x), seed=seed, shape=(rows, cols), scale=scale)


def _attention_tensors():
    return tuple(
        Tensor(4, shape_options=(None, None, {"constexpr": True}, {"constexpr": True, "upper_bound": 128}))
        for _ in range(4)
    )


def run_attention(shape, seed, blocks, is_causal, scale=None):
    q, k, v = oi.attention_inputs(shape, seed)
    out = torch.empty(shape, dtype=torch.float16)
    q_, k_, v_, o_ = _attention_tensors()
    if scale is None:
        kernel = ninetoothed.make(
            functools.partial(ref_attention.arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1]),
            ref_attention.application,
            (q_, k_, v_, Tensor(0, constexpr=True), o_),
        )
        kernel(t(q), t(k), t(v), is_causal, out)
    else:
        # The reference's application with one extra run-time scalar folded
        # into the same rounding point as its log2(e) pre-scale.
        def arrangement(q, k, v, scale, is_causal, o):
            qa, ka, va, c, oa = ref_attention.arrangement(
                q, k, v, is_causal, o, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1]
            )
            return qa, ka, va, scale, c, oa

        def application(q, k, v, scale, is_causal, o):
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

        kernel = ninetoothed.make(
            arrangement, application, (q_, k_, v_, Tensor(0), Tensor(0, constexpr=True), o_)
        )
        kernel(t(q), t(k), t(v), float(scale), is_causal, out)
    return dict(out=out.numpy(), inputs=checksum(q, k, v), seed=seed, shape=shape, blocks=blocks,
                is_causal=is_causal, scale=-1.0 if scale is None else float(scale))


def run_conv2d(xshape, wshape, seed, padding, blocks):
    x, w = oi.conv2d_inputs(xshape, wshape, seed)
    n, _, h, wd = xshape
    kout, _, r, s = wshape
    p = h + 2 * padding[0] - r + 1
    q = wd + 2 * padding[1] - s + 1
    out = torch.empty((n, kout, p, q), dtype=torch.float16)
    kernel = ninetoothed.make(
        functools.partial(ref_conv2d.arrangement, enable_padding=True,
                          BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1], BLOCK_SIZE_K=blocks[2]),
        ref_matmul.application,
        (Tensor(4), Tensor(4, shape_options={"constexpr": True}), Tensor(4)),
    )
    kernel(t(x), t(w), out, padding_h=padding[0], padding_w=padding[1])
    return dict(out=out.numpy(), inputs=checksum(x, w), seed=seed, xshape=xshape, wshape=wshape,
                padding=padding, blocks=blocks)


def run_max_pool2d(shape, window, seed, ceil_mode, block):
    x = ok.normal(seed, shape, np.float16)
    n, c, h, w = shape
    r, s = window
    div = (lambda a, b: -(-a // b)) if ceil_mode else (lambda a, b: a // b)
    out = torch.empty((n, c, div(h - r, r) + 1, div(w - s, s) + 1), dtype=torch.float16)

    def arrangement(input, output):
        # tests/test_max_pool2d.py:13-33 with the meta block size bound to a number (no auto-tuning here)
        window_height = Symbol("WINDOW_HEIGHT", constexpr=True, upper_bound=16)
        window_width = Symbol("WINDOW_WIDTH", constexpr=True, upper_bound=16)
        input_arranged = input.tile((1, 1, window_height, window_width), floor_mode=not ceil_mode)
        input_arranged = input_arranged.ravel().flatten(end_dim=4).flatten(start_dim=1).tile((block, -1))
        output_arranged = output.tile((1, 1, 1, 1)).ravel().flatten(end_dim=4).flatten(start_dim=1).tile((block, -1))
        output_arranged.dtype = output_arranged.dtype.squeeze(1)
        return input_arranged, output_arranged

    kernel = ninetoothed.make(arrangement, ref_max_pool2d.application, (Tensor(4, other=float("-inf")), Tensor(4)))
    kernel(t(x), out, WINDOW_HEIGHT=r, WINDOW_WIDTH=s)
    return dict(out=out.numpy(), inputs=checksum(x), seed=seed, shape=shape, window=window, ceil_mode=int(ceil_mode))


def run_bmm():
    """The batched matmul: the arrangement of examples/definitions.py (the matmul tiling under a leading batch
    dimension) compiled and run by the reference, plus its ``Tensor.eval`` index maps."""
    from examples import load_definitions

    kd = load_definitions("ninetoothed")

    def one(batch, m, n, k, seed, blocks):
        a = ok.normal(seed, (batch, m, k), np.float16)
        b = ok.normal(seed + 1000, (batch, k, n), np.float16)
        out = torch.empty((batch, m, n), dtype=torch.float16)
        kernel = ninetoothed.make(
            functools.partial(kd.bmm_arrangement, BLOCK_SIZE_M=blocks[0], BLOCK_SIZE_N=blocks[1], BLOCK_SIZE_K=blocks[2]),
            kd.matmul_application, (Tensor(3), Tensor(3), Tensor(3)))
        kernel(t(a), t(b), out)
        return dict(out=out.numpy(), inputs=checksum(a, b), seed=seed, shape=(batch, m, n, k), blocks=blocks)

    batch, m, n, k = 2, 5, 7, 6
    arranged = kd.bmm_arrangement(*(Tensor(shape=s) for s in ((batch, m, k), (batch, k, n), (batch, m, n))), 2, 3, 4)
    index_maps = {f"arg{i}": np.asarray(ninetoothed.eval(x)) for i, x in enumerate(arranged)}
    return {"square": one(3, 128, 128, 64, 25, (64, 64, 32)), "ragged": one(2, 100, 70, 90, 26, (32, 32, 32)),
            "index_maps": index_maps}


def run_arrangements():
    """Index maps (``Tensor.eval``, src/ninetoothed/eval.py:15-58) of the reference's
    arrangements on small concrete shapes; -1 marks masked positions."""
    import tests.test_matmul as rm

    def tensors(*shapes, **kw):
        return tuple(Tensor(shape=s, **kw) for s in shapes)

    def maps(arranged):
        return {f"arg{i}": np.asarray(ninetoothed.eval(t)) for i, t in enumerate(arranged)
                if isinstance(t, Tensor) and t.ndim > 0}

    cases = {}
    m, n, k = 5, 7, 6
    cases["matmul"] = maps(rm.arrangement(*tensors((m, k), (k, n), (m, n)), 2, 3, 4))
    cases["addmm"] = maps(ref_addmm.arrangement(*tensors((m, n), (m, k), (k, n)), Tensor(0), Tensor(0),
                                                *tensors((m, n)), 2, 3, 4))
    cases["softmax"] = maps(tuple(t.tile((1, 8)) for t in tensors((5, 7), (5, 7))))
    shape = (2, 3, 7, 4)
    q, kk, v, o = tensors(shape, shape, shape, shape)
    cases["attention"] = maps(ref_attention.arrangement(q, kk, v, Tensor(0, constexpr=True), o, 3, 2))
    xs, ws = (2, 3, 5, 6), (4, 3, 3, 2)
    for ph, pw in ((0, 0), (1, 2)):
        ys = (2, 4, 5 + 2 * ph - 3 + 1, 6 + 2 * pw - 2 + 1)
        x, w, y = tensors(xs, ws, ys)
        # tests/test_conv2d.py:22-48 with the padding symbols bound to numbers
        x = x.pad(((0, 0), (0, 0), (ph, ph), (pw, pw)))
        tiled = x.tile((1, *w.shape[1:]), strides=(-1, -1, 1, 1)).squeeze(1)
        tiled.dtype = tiled.dtype.squeeze(0)
        a = tiled.ravel().flatten(end_dim=3).flatten(start_dim=1)
        b = w.flatten(start_dim=1).permute((1, 0))
        c = y.permute((0, 2, 3, 1)).flatten(end_dim=3)
        cases[f"conv2d_pad_{ph}_{pw}"] = maps(rm.arrangement(a, b, c, 4, 2, 5))
    # tests/test_max_pool2d.py:13-33 with the window and block symbols bound to numbers (3 x 2 windows,
    # blocks of 4 outputs), floor and ceil tiling
    for ceil_mode in (False, True):
        div = (lambda a, b: -(-a // b)) if ceil_mode else (lambda a, b: a // b)
        xs = (2, 3, 7, 8)
        ys = (2, 3, div(7 - 3, 3) + 1, div(8 - 2, 2) + 1)
        x, y = tensors(xs, ys)
        x = x.tile((1, 1, 3, 2), floor_mode=not ceil_mode).ravel().flatten(end_dim=4).flatten(start_dim=1).tile((4, -1))
        y = y.tile((1, 1, 1, 1)).ravel().flatten(end_dim=4).flatten(start_dim=1).tile((4, -1))
        y.dtype = y.dtype.squeeze(1)
        cases[f"max_pool2d_{'ceil' if ceil_mode else 'floor'}"] = maps((x, y))
    return cases


def save(name, cases):
    flat = {}
    for case, fields in cases.items():
        for key, value in fields.items():
            flat[f"{case}/{key}"] = np.asarray(value)
    np.savez_compressed(HERE / f"{name}.npz", **flat)
    print(f"wrote {name}.npz: {sorted(cases)}", flush=True)


def main():
    t0 = time.time()
    if "bmm" in sys.argv[2:]:
        save("bmm", run_bmm())
        return
    save("arrangements", run_arrangements())
    if "arrangements" in sys.argv[2:]:
        return
    save("matmul_e5m2", {
        "square_128": run_matmul_e5m2(128, 128, 128, 19, (32, 32, 32)),
        "ragged": run_matmul_e5m2(72, 40, 96, 20, (32, 32, 32)),
    })
    print("matmul_e5m2", time.time() - t0, flush=True)
    save("max_pool2d", {
        f"w{r}x{s}_{'ceil' if ceil else 'floor'}": run_max_pool2d((2, 3, 16, 20), (r, s), 18, ceil, 32)
        for r, s in ((3, 3), (2, 2), (3, 2)) for ceil in (False, True)
    })
    print("max_pool2d", time.time() - t0, flush=True)
    if "max_pool2d" in sys.argv[2:]:
        return
    save("matmul", {
        "cfg1_512": run_matmul(512, 512, 512, 0, (64, 64, 64)),
        "ragged": run_matmul(100, 70, 90, 10, (32, 32, 32)),
    })
    print("matmul", time.time() - t0, flush=True)
    save("addmm", {
        "unit": run_addmm(128, 128, 128, 1, (64, 64, 64), 1.0, 1.0),
        "scaled_ragged": run_addmm(96, 80, 112, 11, (32, 32, 32), -1.3, 0.7),
    })
    save("softmax", {
        "fp32_781": run_softmax_fp32(37, 781, 12),
        "fp16_8192": run_softmax_fp16(16, 8192, 2, 4.0),
        "fp16_1000": run_softmax_fp16(5, 1000, 16, 4.0),
    })
    print("softmax", time.time() - t0, flush=True)
    save("attention", {
        "d64": run_attention((1, 2, 256, 64), 13, (64, 32), False),
        "d64_causal": run_attention((1, 2, 256, 64), 13, (64, 32), True),
        "s1": run_attention((2, 4, 1, 64), 17, (64, 32), False),
        "s1_causal": run_attention((2, 4, 1, 64), 17, (64, 32), True),
        "ragged_d128_causal": run_attention((1, 1, 200, 128), 14, (64, 64), True),
        "scaled_d128": run_attention((1, 2, 256, 128), 3, (64, 64), False, scale=ok.default_scale(128)),
        "scaled_d128_causal": run_attention((1, 2, 256, 128), 3, (64, 64), True, scale=ok.default_scale(128)),
    })
    print("attention", time.time() - t0, flush=True)
    save("conv2d", {
        f"pad_{ph}_{pw}": run_conv2d((2, 16, 10, 10), (32, 16, 3, 3), 15, (ph, pw), (32, 32, 32))
        for ph, pw in ((0, 0), (1, 1), (0, 1), (2, 0))
    })
    print("done", time.time() - t0, flush=True)


if __name__ == "__main__":
    main()
