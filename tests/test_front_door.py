"""CPU tests of the host side: meta-operations, recognition, call binding.

The arrangement index maps are pinned against ``Tensor.eval`` of the reference
(fixtures in tests/golden/arrangements.npz, produced by tests/golden/generate.py),
in the spirit of the reference's tests/test_eval.py and tests/test_debugging.py.
"""

import functools

import numpy as np
import pytest

import ninetoothed_b200 as ninetoothed
import ninetoothed_b200.language as ntl
from ninetoothed_b200 import Symbol, Tensor, UnsupportedKernelError
from ninetoothed_b200 import recognition
from ninetoothed_b200.tensor import ProbeScope

from examples import definitions as kd
from conftest import load_golden


def _bound(*shapes, **kw):
    return tuple(Tensor(len(s), **kw).instantiate(s) for s in shapes)


def _assert_maps(arranged, golden_case):
    checked = 0
    for i, t in enumerate(arranged):
        key = f"arg{i}"
        if key in golden_case:
            assert np.array_equal(t.index_map(), golden_case[key]), key
            checked += 1
    assert checked == len(golden_case)


def test_matmul_and_addmm_index_maps_match_reference_eval():
    g = load_golden("arrangements")
    m, n, k = 5, 7, 6
    _assert_maps(kd.matmul_arrangement(*_bound((m, k), (k, n), (m, n)), 2, 3, 4), g["matmul"])
    c, a, b, out = _bound((m, n), (m, k), (k, n), (m, n))
    _assert_maps(kd.addmm_arrangement(c, a, b, Tensor(0), Tensor(0), out, 2, 3, 4), g["addmm"])


def test_bmm_index_maps_match_reference_eval_and_the_pair_is_recognised():
    g = load_golden("bmm")["index_maps"]
    batch, m, n, k = 2, 5, 7, 6
    _assert_maps(kd.bmm_arrangement(*_bound((batch, m, k), (batch, k, n), (batch, m, n)), 2, 3, 4), g)
    a_map, b_map, c_map = recognition.bmm_maps(batch, m, n, k, 2, 3, 4)
    assert np.array_equal(a_map, g["arg0"]) and np.array_equal(b_map, g["arg1"]) and np.array_equal(c_map, g["arg2"])
    assert kd.make_bmm().op == "bmm"
    with pytest.raises(UnsupportedKernelError):  # the batched tiling under a body that is not the matmul
        ninetoothed.make(kd.bmm_arrangement, kd.max_pool2d_application, (Tensor(3), Tensor(3), Tensor(3)))


def test_softmax_and_attention_index_maps_match_reference_eval():
    g = load_golden("arrangements")
    x, y = _bound((5, 7), (5, 7))
    _assert_maps((x.tile((1, 8)), y.tile((1, 8))), g["softmax"])
    shape = (2, 3, 7, 4)
    q, k, v, o = _bound(shape, shape, shape, shape)
    _assert_maps(kd.attention_arrangement(q, k, v, Tensor(0, constexpr=True), o, 3, 2), g["attention"])


@pytest.mark.parametrize("ph, pw", [(0, 0), (1, 2)])
def test_conv2d_index_maps_match_reference_eval(ph, pw):
    g = load_golden("arrangements")[f"conv2d_pad_{ph}_{pw}"]
    xs, ws = (2, 3, 5, 6), (4, 3, 3, 2)
    ys = (2, 4, 5 + 2 * ph - 3 + 1, 6 + 2 * pw - 2 + 1)
    with ProbeScope({"padding_h": ph, "padding_w": pw}):
        arranged = kd.conv2d_arrangement(*_bound(xs, ws, ys), enable_padding=True,
                                         BLOCK_SIZE_M=4, BLOCK_SIZE_N=2, BLOCK_SIZE_K=5)
    _assert_maps(arranged, g)


@pytest.mark.parametrize("ceil_mode", [False, True])
def test_max_pool2d_index_maps_match_reference_eval(ceil_mode):
    g = load_golden("arrangements")[f"max_pool2d_{'ceil' if ceil_mode else 'floor'}"]
    in_map, out_map, (p, q) = recognition.max_pool2d_maps((2, 3, 7, 8), (3, 2), ceil_mode, 4)
    assert np.array_equal(in_map, g["arg0"]) and np.array_equal(out_map, g["arg1"])
    with ProbeScope({"WINDOW_HEIGHT": 3, "WINDOW_WIDTH": 2, "BLOCK_SIZE": 4}):
        arranged = kd.max_pool2d_arrangement(*_bound((2, 3, 7, 8), (2, 3, p, q)), ceil_mode=ceil_mode)
    _assert_maps(arranged, g)


def test_canonical_maps_equal_reference_eval():
    """The kernels' own tilings, built without the meta-operations, are the same maps."""
    g = load_golden("arrangements")
    ident = recognition.identity
    a, b, c = recognition.matmul_maps(ident((5, 6)), ident((6, 7)), ident((5, 7)), 2, 3, 4)
    assert np.array_equal(a, g["matmul"]["arg0"]) and np.array_equal(b, g["matmul"]["arg1"])
    assert np.array_equal(c, g["matmul"]["arg2"])
    assert np.array_equal(recognition.softmax_map(5, 7, 8), g["softmax"]["arg0"])
    q_map, kv_map = recognition.attention_maps((2, 3, 7, 4), 3, 2)
    assert np.array_equal(q_map, g["attention"]["arg0"]) and np.array_equal(kv_map, g["attention"]["arg1"])
    am, bm, cm, _ = recognition.conv2d_index_matrices((2, 3, 5, 6), (4, 3, 3, 2), 1, 2)
    a, b, c = recognition.matmul_maps(am, bm, cm, 4, 2, 5)
    gc = g["conv2d_pad_1_2"]
    assert np.array_equal(a, gc["arg0"]) and np.array_equal(b, gc["arg1"]) and np.array_equal(c, gc["arg2"])


@pytest.mark.parametrize("factory, op, constexprs", [
    (kd.make_matmul, "matmul", ()),
    (kd.make_addmm, "addmm", ()),
    (kd.make_softmax, "softmax", ("BLOCK_SIZE",)),
    (kd.make_softmax_fp32_math, "softmax", ("BLOCK_SIZE",)),
    (kd.make_attention, "attention", ()),
    (kd.make_scaled_attention, "attention_scaled", ()),
    (kd.make_conv2d, "conv2d", ("padding_h", "padding_w")),
    (functools.partial(kd.make_conv2d, enable_padding=False), "conv2d", ()),
    (functools.partial(kd.make_max_pool2d, ceil_mode=False), "max_pool2d", ("WINDOW_HEIGHT", "WINDOW_WIDTH")),
    (functools.partial(kd.make_max_pool2d, ceil_mode=True), "max_pool2d", ("WINDOW_HEIGHT", "WINDOW_WIDTH")),
])
def test_reference_definitions_are_recognised(factory, op, constexprs):
    handle = factory()
    assert handle.op == op
    assert handle.constexpr_names == constexprs


def test_readme_matmul_with_fixed_block_sizes():
    arrangement = functools.partial(kd.matmul_arrangement, BLOCK_SIZE_M=64, BLOCK_SIZE_N=64, BLOCK_SIZE_K=64)
    handle = ninetoothed.make(arrangement, kd.readme_matmul_application, (Tensor(2), Tensor(2), Tensor(2)),
                              num_warps=8, num_stages=3)
    assert handle.op == "matmul"
    assert handle.block_sizes == {"BLOCK_SIZE_M": 64, "BLOCK_SIZE_N": 64, "BLOCK_SIZE_K": 64}


def elementwise_arrangement(a, b, c):
    return a.tile((4, 4)), b.tile((4, 4)), c.tile((4, 4))


def elementwise_application(a, b, c):
    c = a + b  # noqa: F841


def transposed_matmul_arrangement(lhs, rhs, output):
    return kd.matmul_arrangement(lhs.permute((1, 0)), rhs, output)


def test_other_kernels_are_rejected_loudly():
    tensors = (Tensor(2), Tensor(2), Tensor(2))
    with pytest.raises(UnsupportedKernelError):
        ninetoothed.make(elementwise_arrangement, elementwise_application, tensors)
    with pytest.raises(UnsupportedKernelError):  # right tiling, wrong body
        ninetoothed.make(kd.matmul_arrangement, elementwise_application, tensors)
    with pytest.raises(UnsupportedKernelError):  # right body, different tiling
        ninetoothed.make(elementwise_arrangement, kd.matmul_application, tensors)
    with pytest.raises(UnsupportedKernelError):  # softmax body under the matmul tiling
        ninetoothed.make(kd.matmul_arrangement, kd.addmm_application, tensors)
    with pytest.raises(ValueError):
        ninetoothed.make(kd.matmul_arrangement, kd.matmul_application, tensors, caller="cpu")
    with pytest.raises(UnsupportedKernelError):
        ninetoothed.make(transposed_matmul_arrangement, kd.matmul_application, (Tensor(2), Tensor(2), Tensor(2)))


# Bodies one edit away from an implemented one: each computes something else, so each must be rejected
# (a handle that ran the plain kernel for them would return wrong numbers without a word).
def _matmul_with_an_affine_tail(lhs, rhs, output):
    accumulator = ntl.zeros(output.shape, dtype=ntl.float32)
    for k in range(lhs.shape[0]):
        accumulator += ntl.dot(lhs[k], rhs[k])
    output = (accumulator * 0.5 - 3.0).to(ntl.float16)  # noqa: F841


def _matmul_with_swapped_operands(lhs, rhs, output):
    accumulator = ntl.zeros(output.shape, dtype=ntl.float32)
    for k in range(lhs.shape[0]):
        accumulator += ntl.dot(rhs[k], lhs[k])
    output = accumulator.to(ntl.float16)  # noqa: F841


def _softmax_with_a_tail(input_row, output_row):
    row_minus_max = input_row - ntl.max(input_row)
    numerator = ntl.exp(row_minus_max)
    denominator = ntl.sum(numerator)
    output_row = numerator / denominator * 2.0 + denominator  # noqa: F841


def _maximum_along_the_other_axis(input, output):
    output = ntl.max(input, axis=0)  # noqa: F841


def _addmm_with_swapped_scalars(input, mat1, mat2, beta, alpha, output):
    matmul_output = ntl.zeros(output.shape, dtype=ntl.float32)
    kd.matmul_application(mat1, mat2, matmul_output)
    output = alpha * input + beta * matmul_output  # noqa: F841


def _matmul_renamed(a, b, c):
    """Same body as the matmul application under other names: accepted."""
    acc = ntl.zeros(c.shape, dtype=ntl.float32)
    for step in range(a.shape[0]):
        acc += ntl.dot(a[step], b[step])
    c = acc.to(ntl.bfloat16)  # noqa: F841


@pytest.mark.parametrize("body", [_matmul_with_an_affine_tail, _matmul_with_swapped_operands, _softmax_with_a_tail,
                                  _maximum_along_the_other_axis, _addmm_with_swapped_scalars])
def test_near_miss_applications_are_rejected(body):
    with pytest.raises(UnsupportedKernelError):
        recognition.recognise_application(body)


def test_application_matching_ignores_names_docstrings_and_inlining():
    assert recognition.recognise_application(_matmul_renamed) == "matmul"
    assert recognition.recognise_application(kd.matmul_application) == "matmul"
    assert recognition.recognise_application(kd.readme_matmul_application) == "matmul"
    assert recognition.recognise_application(kd.addmm_application) == "addmm"  # calls the matmul application
    assert recognition.recognise_application(kd.attention_application) == "attention"
    assert recognition.recognise_application(kd.scaled_attention_application) == "attention_scaled"
    assert recognition.recognise_application(kd.max_pool2d_application) == "row_max"
    assert recognition.recognise_application(_softmax_body) == "softmax"


def test_softmax_needs_minus_infinity_padding():
    BLOCK_SIZE = Symbol("BLOCK_SIZE", constexpr=True)

    def arrangement(x, y):
        return x.tile((1, BLOCK_SIZE)), y.tile((1, BLOCK_SIZE))

    with pytest.raises(UnsupportedKernelError):
        ninetoothed.make(arrangement, _softmax_body, (Tensor(2), Tensor(2)))


def _softmax_body(input_row, output_row):
    row_minus_max = input_row - ntl.max(input_row)
    numerator = ntl.exp(row_minus_max)
    denominator = ntl.sum(numerator)
    output_row = numerator / denominator  # noqa: F841


def test_call_binding_errors_do_not_reach_the_device():
    handle = kd.make_conv2d()
    with pytest.raises(TypeError):
        handle(1, 2)  # too few tensors
    with pytest.raises(TypeError):
        handle(1, 2, 3, stride=2)  # unknown constexpr
    with pytest.raises(TypeError):
        handle(1, 2, 3, padding_h=1)  # padding_w missing
    softmax = kd.make_softmax()
    with pytest.raises(TypeError):
        softmax(1, 2)  # BLOCK_SIZE missing


def test_symbol_arithmetic_and_bounds():
    bs = ninetoothed.block_size(lower_bound=64, upper_bound=128)
    assert bs.meta and bs.constexpr and (bs.lower_bound, bs.upper_bound) == (64, 128)
    default = Symbol("X", meta=True)
    assert (default.lower_bound, default.upper_bound, default.power_of_two) == (32, 1024, True)
    c = Symbol("padding", constexpr=True)
    assert (2 * c + 1).evaluate({"padding": 3}) == 7
    assert (c // 2).evaluate({"padding": 7}) == 3
    with pytest.raises(ValueError):
        Symbol(3, meta=True)


def test_meta_operations_on_partial_tiles_and_strides():
    (x,) = _bound((5, 7))
    tiled = x.tile((2, 3))
    assert tiled.levels() == [(3, 3), (2, 3)]
    assert tiled.index_map()[2, 2, 1, 0] == -1  # row 5 is out of range
    assert tiled.index_map()[2, 2, 0, 0] == 4 * 7 + 6
    assert tiled.index_map()[2, 2, 0, 1] == -1  # column 7 is out of range
    windows = x.tile((2, 2), strides=(1, 1))
    assert windows.levels() == [(4, 6), (2, 2)]
    assert windows.index_map()[3, 5].tolist() == [[3 * 7 + 5, 3 * 7 + 6], [4 * 7 + 5, 4 * 7 + 6]]
    dilated = x.tile((2, 2), strides=(1, 1), dilation=(2, 3))
    assert dilated.index_map()[0, 0].tolist() == [[0, 3], [14, 17]]
    assert x.unsqueeze(1).shape == (5, 1, 7)
    assert x.permute((1, 0)).index_map()[2, 3] == 3 * 7 + 2
    assert x.pad(((1, 0), (0, 2))).index_map()[0, 0] == -1


# ---------------------------------------------------------------- build(): dispatch over configurations
def _conv2d_build(sizes, configs, **kwargs):
    import functools

    import ninetoothed_b200 as ninetoothed
    from examples import definitions as kd

    premake = functools.partial(kd.conv2d_premake, **sizes, dtype=ninetoothed.float16)
    return ninetoothed.build(premake, configs, caller="cuda", kernel_name="conv2d_test", output_dir="unused", **kwargs)


def test_build_dispatches_on_the_trailing_configuration_values():
    """tests/test_aot.py:256-301 of the reference: two block-size configurations, the call passes
    premake's bound arguments (sizes, dtype, block sizes) after the tensors."""
    from ninetoothed_b200 import dispatch

    sizes = {"n": None, "c": None, "h": None, "w": None, "k": None, "r": None, "s": None}
    configs = (
        ((), {"block_size_m": 64, "block_size_n": 64, "block_size_k": 64}, {}),
        ((), {"block_size_m": 128, "block_size_n": 32, "block_size_k": 64}, {}),
    )
    kernel = _conv2d_build(sizes, configs)
    assert [v.handle.op for v in kernel.variants] == ["conv2d", "conv2d"]
    assert kernel.num_tensor_params == 3
    assert kernel.param_names == ("n_", "c_", "h_", "w_", "k_", "r_", "s_", "dtype_", "block_size_m_", "block_size_n_",
                                  "block_size_k_")
    # dtype tags and None are converted like the reference does (float16 -> 8, None -> 0)
    assert kernel.variants[1].combination == {"n_": 0, "c_": 0, "h_": 0, "w_": 0, "k_": 0, "r_": 0, "s_": 0,
                                              "dtype_": 8, "block_size_m_": 128, "block_size_n_": 32,
                                              "block_size_k_": 64}

    launched = []
    for index, variant in enumerate(kernel.variants):
        variant.handle = lambda *tensors, index=index: launched.append((index, tensors))
    import ninetoothed_b200 as ninetoothed

    kernel("x", "w", "y", *sizes.values(), ninetoothed.float16, 128, 32, 64)
    kernel("x", "w", "y", *sizes.values(), ninetoothed.float16, 64, 64, 64)
    assert launched == [(1, ("x", "w", "y")), (0, ("x", "w", "y"))]
    with pytest.raises(dispatch.KernelLaunchError) as info:
        kernel("x", "w", "y", *sizes.values(), ninetoothed.float16, 32, 32, 32)
    assert info.value.error_code == 1
    with pytest.raises(TypeError):
        kernel("x", "w", "y", 64, 64, 64)


def test_build_meta_parameters_are_not_passed_by_the_caller_and_lazy_defers():
    sizes = {"n": 4, "c": 64, "h": 16, "w": 16, "k": 512, "r": 3, "s": 3}
    configs = tuple(((), {"block_size_m": bm, "block_size_n": 64, "block_size_k": 64}, {"num_warps": 4})
                    for bm in (64, 128))
    kernel = _conv2d_build(sizes, configs, meta_parameters=("block_size_m", "block_size_n", "block_size_k", "num_warps"))
    launched = []
    kernel.variants[0].handle = lambda *tensors: launched.append(tensors)
    import ninetoothed_b200 as ninetoothed

    kernel("x", "w", "y", *sizes.values(), ninetoothed.float16)
    assert launched == [("x", "w", "y")]

    calls = []

    def premake(**kwargs):
        calls.append(kwargs)
        from examples import definitions as kd

        return kd.conv2d_premake(**kwargs)

    lazy = ninetoothed.build(premake, (((), {"dtype": ninetoothed.float16}, {}),), kernel_name="lazy_conv2d",
                             output_dir="unused", lazy=True)
    assert calls == []
    with pytest.raises(Exception):
        lazy("x", "w", "y")  # wrong arity reaches the dispatcher only after the deferred build ran
    assert len(calls) == 1


def test_build_rejects_what_make_rejects():
    import ninetoothed_b200 as ninetoothed
    from ninetoothed_b200 import Tensor

    def premake(block_size=64):
        def arrangement(x, y, BLOCK_SIZE=block_size):
            return x.tile((BLOCK_SIZE,)), y.tile((BLOCK_SIZE,))

        def application(x, y):
            y = x + x  # noqa: F841

        return arrangement, application, (Tensor(1), Tensor(1))

    with pytest.raises(ninetoothed.UnsupportedKernelError):
        ninetoothed.build(premake, (((), {}, {}),), kernel_name="double", output_dir="unused")


def test_max_pool2d_mode_is_read_from_the_tiling_and_other_must_be_minus_infinity():
    assert kd.make_max_pool2d(False)._ceil_mode is False and kd.make_max_pool2d(True)._ceil_mode is True
    with pytest.raises(UnsupportedKernelError, match="-inf"):
        ninetoothed.make(kd.max_pool2d_arrangement, kd.max_pool2d_application, (Tensor(4), Tensor(4)))
    with pytest.raises(UnsupportedKernelError):  # the window arrangement under another application
        ninetoothed.make(kd.max_pool2d_arrangement, kd.matmul_application, (Tensor(4, other=float("-inf")), Tensor(4)))
