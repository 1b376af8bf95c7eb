"""Activation modules (crates/axonml-nn/src/activation.rs:21-406).  GELU is the tanh
approximation, as in the reference; Softmax/LogSoftmax are dim-aware (the reference normalises the
whole tensor, ops/mod.rs:134-158, which is not reproduced)."""
from __future__ import annotations

import torch

from ..ops import elementwise as E
from ..ops import loss as L
from .module import Module


class _Act(Module):
    @classmethod
    def new(cls, *a): return cls(*a)


class _KernelAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, p0):
        y = E.unary(x, op, p0)
        ctx.op, ctx.p0 = op, p0
        ctx.save_for_backward(y if op in ("sigmoid", "tanh") else x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (s,) = ctx.saved_tensors
        return E.act_backward(dy.contiguous(), s, ctx.op, ctx.p0), None, None


def _act(x, op, p0=0.0):
    if E.kernel_ok(x):
        return _KernelAct.apply(x, op, p0)
    return E._UNARY_REF[op](x, p0, 0.0)


class ReLU(_Act):
    def forward(self, x): return _act(x, "relu")


class LeakyReLU(_Act):
    def __init__(self, negative_slope: float = 0.01):
        super().__init__()
        self.negative_slope = negative_slope

    @classmethod
    def with_slope(cls, slope: float): return cls(slope)

    def forward(self, x): return _act(x, "leaky_relu", self.negative_slope)


class Sigmoid(_Act):
    def forward(self, x): return _act(x, "sigmoid")


class Tanh(_Act):
    def forward(self, x): return _act(x, "tanh")


class GELU(_Act):
    def forward(self, x): return _act(x, "gelu")


class SiLU(_Act):
    def forward(self, x): return _act(x, "silu")


class ELU(_Act):
    def __init__(self, alpha: float = 1.0):
        super().__init__()
        self.alpha = alpha

    @classmethod
    def with_alpha(cls, alpha: float): return cls(alpha)

    def forward(self, x): return _act(x, "elu", self.alpha)


class Identity(_Act):
    def forward(self, x): return x


class Softmax(_Act):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x): return L.softmax(x, self.dim)


class LogSoftmax(_Act):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x): return L.log_softmax(x, self.dim)
