"""Pooling layers (crates/axonml-nn/src/layers/pooling.rs:22-383): ``new(k)`` uses stride = k and
no padding; ``with_options(k, stride, padding)``."""
from __future__ import annotations

import torch.nn.functional as F

from ..module import Module


class _Pool(Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.kernel_size = kernel_size
        self.stride = kernel_size if stride is None else stride
        self.padding = padding

    @classmethod
    def new(cls, kernel_size): return cls(kernel_size)

    @classmethod
    def with_options(cls, kernel_size, stride, padding): return cls(kernel_size, stride, padding)


class MaxPool1d(_Pool):
    def forward(self, x): return F.max_pool1d(x, self.kernel_size, self.stride, self.padding)


class MaxPool2d(_Pool):
    def forward(self, x):
        k, st, p = self.kernel_size, self.stride, self.padding
        if x.dim() == 4 and x.is_cuda and isinstance(k, int) and isinstance(st, int) and isinstance(p, int):
            from ...ops.batchnorm import max_pool2d
            return max_pool2d(x, k, st, p)
        return F.max_pool2d(x, k, st, p)


class AvgPool1d(_Pool):
    """Mean over each window; padded positions do not count (pooling.rs:120-200)."""

    def forward(self, x):
        from ...ops.pool import avg_pool1d
        return avg_pool1d(x, self.kernel_size, self.stride, self.padding)


class AvgPool2d(_Pool):
    """Mean over each window; padded positions do not count (pooling.rs:296-357)."""

    def forward(self, x):
        from ...ops.pool import avg_pool2d
        return avg_pool2d(x, self.kernel_size, self.stride, self.padding)


class AdaptiveAvgPool2d(Module):
    def __init__(self, output_size):
        super().__init__()
        self.output_size = (output_size, output_size) if isinstance(output_size, int) else tuple(output_size)

    @classmethod
    def new(cls, output_size): return cls(output_size)

    @classmethod
    def square(cls, n: int): return cls((n, n))

    def forward(self, x):
        from ...ops.pool import adaptive_avg_pool2d
        return adaptive_avg_pool2d(x, self.output_size)
