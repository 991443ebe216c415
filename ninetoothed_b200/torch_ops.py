"""PyTorch custom ops over the C ABI: ``torch.ops.ninetoothed_b200.*``.

Each op mutates its ``output`` argument in place and returns nothing, which is
the contract of the callable ``ninetoothed.make`` returns
(``src/ninetoothed/jit.py:121-128`` in the reference project: the launch function
writes through the output tensor's pointer).  Only a CUDA implementation is
registered: calling an op with CPU tensors raises, there is no fallback.
"""

from __future__ import annotations

import torch

from ninetoothed_b200 import _capi

_LIBRARY = torch.library.Library("ninetoothed_b200", "DEF")

_LIBRARY.define("matmul(Tensor lhs, Tensor rhs, Tensor(a!) output) -> ()")
_LIBRARY.define("bmm(Tensor lhs, Tensor rhs, Tensor(a!) output) -> ()")
_LIBRARY.define("addmm(Tensor input, Tensor mat1, Tensor mat2, float beta, float alpha, Tensor(a!) output) -> ()")
_LIBRARY.define("softmax(Tensor input, Tensor(a!) output) -> ()")
_LIBRARY.define("attention(Tensor q, Tensor k, Tensor v, bool is_causal, Tensor(a!) o) -> ()")
_LIBRARY.define("attention_scaled(Tensor q, Tensor k, Tensor v, float scale, bool is_causal, Tensor(a!) o) -> ()")
_LIBRARY.define("conv2d(Tensor input, Tensor filter, Tensor(a!) output, int padding_h, int padding_w) -> ()")
_LIBRARY.define("max_pool2d(Tensor input, Tensor(a!) output, int window_height, int window_width, bool ceil_mode) -> ()")


def _matmul(lhs, rhs, output):
    _capi.matmul(lhs, rhs, output)


def _bmm(lhs, rhs, output):
    _capi.bmm(lhs, rhs, output)


def _addmm(input, mat1, mat2, beta, alpha, output):
    _capi.addmm(input, mat1, mat2, beta, alpha, output)


def _softmax(input, output):
    _capi.softmax(input, output)


def _attention(q, k, v, is_causal, o):
    _capi.attention(q, k, v, is_causal, o)


def _attention_scaled(q, k, v, scale, is_causal, o):
    _capi.attention(q, k, v, is_causal, o, scale=scale)


def _conv2d(input, filter, output, padding_h, padding_w):
    _capi.conv2d(input, filter, output, padding_h, padding_w)


def _max_pool2d(input, output, window_height, window_width, ceil_mode):
    _capi.max_pool2d(input, output, window_height, window_width, ceil_mode)


_LIBRARY.impl("matmul", _matmul, "CUDA")
_LIBRARY.impl("bmm", _bmm, "CUDA")
_LIBRARY.impl("addmm", _addmm, "CUDA")
_LIBRARY.impl("softmax", _softmax, "CUDA")
_LIBRARY.impl("attention", _attention, "CUDA")
_LIBRARY.impl("attention_scaled", _attention_scaled, "CUDA")
_LIBRARY.impl("conv2d", _conv2d, "CUDA")
_LIBRARY.impl("max_pool2d", _max_pool2d, "CUDA")

ops = torch.ops.ninetoothed_b200
