"""Backward functions of the basic operations, by name.

Parity: crates/axonml-autograd/src/functions/{basic,activation,linalg,loss}.rs (``AddBackward``,
``SubBackward``, ``MulBackward``, ``DivBackward``, ``NegBackward``, ``PowBackward``,
``SumBackward``, ``MeanBackward``, ``NarrowBackward``; ``ReluBackward``, ``SigmoidBackward``,
``TanhBackward``, ``GeluBackward``, ``LeakyReluBackward``, ``SoftmaxBackward``;
``MatMulBackward``, ``TransposeBackward``, ``ReshapeBackward``, ``ViewBackward``,
``SqueezeBackward``, ``UnsqueezeBackward``; the six loss backwards) and grad_fn.rs:112-140
(``AccumulateGrad``).

Every class is a ``GradientFunction``: ``X.call(*inputs, **options)`` runs the forward outside the
tape and records a node whose backward is the class's ``apply``.  The tape's own operators do not
go through these (torch differentiates them); they are the reference formulas, usable as building
blocks for operations written outside the tape and checked against the tape in the tests.
Gradients of broadcast operands are summed back to the operand's shape."""
from __future__ import annotations

import math

import torch

from .graph import GradientFunction


def sum_to_shape(grad: torch.Tensor, shape) -> torch.Tensor:
    """Reduces a gradient of a broadcast result back to the operand's ``shape``."""
    shape = tuple(shape)
    if tuple(grad.shape) == shape:
        return grad
    lead = grad.dim() - len(shape)
    if lead > 0:
        grad = grad.sum(dim=tuple(range(lead)))
    dims = tuple(i for i, (g, s) in enumerate(zip(grad.shape, shape)) if s == 1 and g != 1)
    if dims:
        grad = grad.sum(dim=dims, keepdim=True)
    return grad.reshape(shape)


# ------------------------------------------------------------------------------------------ basic
class _Binary(GradientFunction):
    def forward(self, a, b):
        self.shapes = (a.shape, b.shape)
        self.save_for_backward(a, b)
        return self.op(a, b)


class AddBackward(_Binary):
    op = staticmethod(torch.add)
    def apply(self, g): return sum_to_shape(g, self.shapes[0]), sum_to_shape(g, self.shapes[1])


class SubBackward(_Binary):
    op = staticmethod(torch.sub)
    def apply(self, g): return sum_to_shape(g, self.shapes[0]), sum_to_shape(-g, self.shapes[1])


class MulBackward(_Binary):
    op = staticmethod(torch.mul)

    def apply(self, g):
        a, b = self.saved_tensors
        return sum_to_shape(g * b, self.shapes[0]), sum_to_shape(g * a, self.shapes[1])


class DivBackward(_Binary):
    op = staticmethod(torch.div)

    def apply(self, g):
        a, b = self.saved_tensors
        return sum_to_shape(g / b, self.shapes[0]), sum_to_shape(-g * a / (b * b), self.shapes[1])


class NegBackward(GradientFunction):
    def forward(self, x): return -x
    def apply(self, g): return (-g,)


class PowBackward(GradientFunction):
    def __init__(self, exponent: float = 2.0): self.exponent = float(exponent)

    def forward(self, x):
        self.save_for_backward(x)
        return x ** self.exponent

    def apply(self, g):
        (x,) = self.saved_tensors
        return (g * self.exponent * x ** (self.exponent - 1.0),)


class SumBackward(GradientFunction):
    def forward(self, x):
        self.input_shape = x.shape
        return x.sum()

    def apply(self, g): return (g.expand(self.input_shape),)


class MeanBackward(GradientFunction):
    def forward(self, x):
        self.input_shape, self.n = x.shape, x.numel()
        return x.mean()

    def apply(self, g): return ((g / self.n).expand(self.input_shape),)


class NarrowBackward(GradientFunction):
    def __init__(self, dim: int = 0, start: int = 0, length: int = 1): self.dim, self.start, self.length = dim, start, length

    def forward(self, x):
        self.input_shape = x.shape
        return x.narrow(self.dim, self.start, self.length)

    def apply(self, g):
        out = g.new_zeros(self.input_shape)
        out.narrow(self.dim, self.start, self.length).copy_(g)
        return (out,)


# ------------------------------------------------------------------------------------- activation
class ReluBackward(GradientFunction):
    def forward(self, x):
        self.save_for_backward(x)
        return x.relu()

    def apply(self, g): return (g * (self.saved_tensors[0] > 0).to(g.dtype),)


class LeakyReluBackward(GradientFunction):
    def __init__(self, negative_slope: float = 0.01): self.slope = float(negative_slope)

    def forward(self, x):
        self.save_for_backward(x)
        return torch.where(x > 0, x, x * self.slope)

    def apply(self, g):
        (x,) = self.saved_tensors
        return (torch.where(x > 0, g, g * self.slope),)


class SigmoidBackward(GradientFunction):
    def forward(self, x):
        y = torch.sigmoid(x)
        self.save_for_backward(y)
        return y

    def apply(self, g):
        (y,) = self.saved_tensors
        return (g * y * (1 - y),)


class TanhBackward(GradientFunction):
    def forward(self, x):
        y = torch.tanh(x)
        self.save_for_backward(y)
        return y

    def apply(self, g):
        (y,) = self.saved_tensors
        return (g * (1 - y * y),)


class GeluBackward(GradientFunction):
    """tanh approximation: 0.5 x (1 + tanh(c (x + 0.044715 x^3))), c = sqrt(2/pi)."""
    C, A = math.sqrt(2.0 / math.pi), 0.044715

    def forward(self, x):
        self.save_for_backward(x)
        return 0.5 * x * (1 + torch.tanh(self.C * (x + self.A * x ** 3)))

    def apply(self, g):
        (x,) = self.saved_tensors
        t = torch.tanh(self.C * (x + self.A * x ** 3))
        return (g * (0.5 * (1 + t) + 0.5 * x * (1 - t * t) * self.C * (1 + 3 * self.A * x * x)),)


class SoftmaxBackward(GradientFunction):
    def __init__(self, dim: int = -1): self.dim = dim

    def forward(self, x):
        y = torch.softmax(x, self.dim)
        self.save_for_backward(y)
        return y

    def apply(self, g):
        (y,) = self.saved_tensors
        return (y * (g - (g * y).sum(self.dim, keepdim=True)),)


# ----------------------------------------------------------------------------------------- linalg
class MatMulBackward(GradientFunction):
    """2-D and batched products; batch dimensions that were broadcast are summed."""

    def forward(self, a, b):
        self.save_for_backward(a, b)
        return a @ b

    def apply(self, g):
        a, b = self.saved_tensors
        if a.dim() == 1 and b.dim() == 1:
            return g * b, g * a
        a2 = a.unsqueeze(0) if a.dim() == 1 else a
        b2 = b.unsqueeze(-1) if b.dim() == 1 else b
        g2 = g.unsqueeze(-2) if a.dim() == 1 else g
        g2 = g2.unsqueeze(-1) if b.dim() == 1 else g2
        ga = sum_to_shape(g2 @ b2.transpose(-1, -2), a2.shape).reshape(a.shape)
        gb = sum_to_shape(a2.transpose(-1, -2) @ g2, b2.shape).reshape(b.shape)
        return ga, gb


class TransposeBackward(GradientFunction):
    def __init__(self, dim0: int = 0, dim1: int = 1): self.dim0, self.dim1 = dim0, dim1
    def forward(self, x): return x.transpose(self.dim0, self.dim1)
    def apply(self, g): return (g.transpose(self.dim0, self.dim1),)


class ReshapeBackward(GradientFunction):
    def __init__(self, shape=(-1,)): self.shape = tuple(shape)

    def forward(self, x):
        self.input_shape = x.shape
        return x.reshape(self.shape)

    def apply(self, g): return (g.reshape(self.input_shape),)


class ViewBackward(ReshapeBackward):
    pass


class SqueezeBackward(GradientFunction):
    def __init__(self, dim: int | None = None): self.dim = dim

    def forward(self, x):
        self.input_shape = x.shape
        return x.squeeze() if self.dim is None else x.squeeze(self.dim)

    def apply(self, g): return (g.reshape(self.input_shape),)


class UnsqueezeBackward(GradientFunction):
    def __init__(self, dim: int = 0): self.dim = dim
    def forward(self, x): return x.unsqueeze(self.dim)
    def apply(self, g): return (g.squeeze(self.dim),)


# ------------------------------------------------------------------------------------------- loss
class _Loss(GradientFunction):
    """``reduction`` is "mean", "sum" or "none"; the target gets no gradient."""

    def __init__(self, reduction: str = "mean"):
        if reduction not in ("mean", "sum", "none"):
            raise ValueError(f"unknown reduction {reduction!r}")
        self.reduction = reduction

    def _reduce(self, per_element, count=None):
        if self.reduction == "none":
            return per_element
        return per_element.sum() if self.reduction == "sum" else per_element.sum() / (count or per_element.numel())

    def _scale(self, g, like, count=None):
        if self.reduction == "none":
            return g
        return g.expand_as(like) if self.reduction == "sum" else (g / (count or like.numel())).expand_as(like)


class MseLossBackward(_Loss):
    def forward(self, x, t):
        self.save_for_backward(x, t)
        return self._reduce((x - t) ** 2)

    def apply(self, g):
        x, t = self.saved_tensors
        return self._scale(g, x) * 2 * (x - t), None


class L1LossBackward(_Loss):
    def forward(self, x, t):
        self.save_for_backward(x, t)
        return self._reduce((x - t).abs())

    def apply(self, g):
        x, t = self.saved_tensors
        return self._scale(g, x) * torch.sign(x - t), None


class SmoothL1LossBackward(_Loss):
    def __init__(self, reduction: str = "mean", beta: float = 1.0):
        super().__init__(reduction)
        self.beta = float(beta)

    def forward(self, x, t):
        self.save_for_backward(x, t)
        d = (x - t).abs()
        return self._reduce(torch.where(d < self.beta, 0.5 * d * d / self.beta, d - 0.5 * self.beta))

    def apply(self, g):
        x, t = self.saved_tensors
        d = x - t
        return self._scale(g, x) * torch.where(d.abs() < self.beta, d / self.beta, torch.sign(d)), None


class BceLossBackward(_Loss):
    """Inputs are probabilities; the logarithms are clamped at -100 like the forward."""
    EPS = 1e-12

    def forward(self, p, t):
        self.save_for_backward(p, t)
        return self._reduce(-(t * torch.log(p).clamp(min=-100) + (1 - t) * torch.log(1 - p).clamp(min=-100)))

    def apply(self, g):
        p, t = self.saved_tensors
        return self._scale(g, p) * (p - t) / (p * (1 - p)).clamp(min=self.EPS), None


class NllLossBackward(_Loss):
    """Input: log-probabilities [N, C]; target: class indices [N]."""

    def forward(self, logp, target):
        self.save_for_backward(logp, target.long())
        return self._reduce(-logp.gather(1, target.long().unsqueeze(1)).squeeze(1))

    def apply(self, g):
        logp, target = self.saved_tensors
        n = logp.shape[0]
        scale = g.reshape(-1, 1) if self.reduction == "none" else (g / n if self.reduction == "mean" else g)
        out = torch.zeros_like(logp)
        out.scatter_(1, target.unsqueeze(1), -1.0)
        return out * scale, None


class CrossEntropyLossBackward(_Loss):
    """Input: logits [N, C]; target: class indices [N].  Gradient = softmax - one-hot."""

    def forward(self, logits, target):
        logp = torch.log_softmax(logits, dim=1)
        self.save_for_backward(logp, target.long())
        return self._reduce(-logp.gather(1, target.long().unsqueeze(1)).squeeze(1))

    def apply(self, g):
        logp, target = self.saved_tensors
        n = logp.shape[0]
        scale = g.reshape(-1, 1) if self.reduction == "none" else (g / n if self.reduction == "mean" else g)
        grad = logp.exp()
        grad.scatter_add_(1, target.unsqueeze(1), -torch.ones_like(grad[:, :1]))
        return grad * scale, None


# --------------------------------------------------------------------------------- accumulation
class GradAccumulator:
    """Shared slot a leaf's gradient is accumulated into (grad_fn.rs:114)."""

    def __init__(self):
        self.value: torch.Tensor | None = None

    def get(self): return self.value
    def clear(self) -> None: self.value = None


class AccumulateGrad(GradientFunction):
    """Terminal node of a leaf: adds every incoming gradient to its accumulator (grad_fn.rs:117-150)."""

    def __init__(self, grad_accumulator: GradAccumulator | None = None):
        self.grad_accumulator = grad_accumulator or GradAccumulator()

    @classmethod
    def new(cls, grad_accumulator): return cls(grad_accumulator)

    def accumulate(self, grad: torch.Tensor) -> None:
        acc = self.grad_accumulator
        acc.value = grad.clone() if acc.value is None else acc.value + grad

    def forward(self, x): return x.clone()

    def apply(self, g):
        self.accumulate(g)
        return (g,)
