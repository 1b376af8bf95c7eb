"""Conv1d / Conv2d (crates/axonml-nn/src/layers/conv.rs:47-87, :202-337): NCHW API, weights
``[cout, cin, k(,k)]`` kaiming-uniform with fan_in = cin*k*k, zero bias.  Unlike the reference the
layers are differentiable.  bf16 inputs on a B200 (channels-last for Conv2d, channel counts that
are multiples of 64 or a thin stem) go through the implicit-GEMM kernels of ``ops.conv_igemm``;
everything else uses the torch convolution."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..module import Module, Parameter


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class Conv1d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding
        bound = math.sqrt(6.0 / (in_channels * kernel_size))
        self.weight = Parameter(torch.empty(out_channels, in_channels, kernel_size).uniform_(-bound, bound))
        if bias:
            self.bias = Parameter(torch.zeros(out_channels))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, cin, cout, k): return cls(cin, cout, k)

    @classmethod
    def with_options(cls, cin, cout, k, stride, padding, bias): return cls(cin, cout, k, stride, padding, bias)

    def forward(self, x):
        from ...ops import conv_igemm as C
        if isinstance(self.stride, int) and isinstance(self.padding, int) and C.conv1d_supported(x, self.weight, self.stride, self.padding):
            return C.conv1d(x, self.weight, self.bias, self.stride, self.padding)
        return F.conv1d(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype),
                        self.stride, self.padding)


class Conv2d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = _pair(kernel_size), _pair(stride), _pair(padding)
        kh, kw = self.kernel_size
        bound = math.sqrt(6.0 / (in_channels * kh * kw))
        self.weight = Parameter(torch.empty(out_channels, in_channels, kh, kw).uniform_(-bound, bound))
        if bias:
            self.bias = Parameter(torch.zeros(out_channels))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, cin, cout, k): return cls(cin, cout, k)

    @classmethod
    def with_options(cls, cin, cout, k, stride, padding, bias): return cls(cin, cout, k, stride, padding, bias)

    def forward(self, x):
        from ...ops import conv_igemm as C
        if C.conv2d_supported(x, self.weight, self.stride, self.padding):
            return C.conv2d(x, self.weight, self.bias, self.stride, self.padding)
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        b = self.bias
        if b is not None and b.dtype != x.dtype:
            b = b.to(x.dtype)
        return F.conv2d(x, w, b, self.stride, self.padding)
