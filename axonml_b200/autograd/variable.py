"""``Variable``: the reference's differentiable tensor handle
(crates/axonml-autograd/src/variable.rs:36-656) as a thin wrapper over a ``torch.Tensor``.  Every
op records in the torch graph - including the ones the reference leaves out of its graph (slice,
expand, gelu, silu, sqrt, softmax, log_softmax, mean_dim, var_dim)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


class Variable:
    __slots__ = ("tensor",)

    def __init__(self, data, requires_grad: bool = False):
        t = data.tensor if isinstance(data, Variable) else torch.as_tensor(data)
        if requires_grad and not t.requires_grad:
            t = t.detach().clone().requires_grad_(True) if not t.is_leaf else t.requires_grad_(True)
        self.tensor = t

    @classmethod
    def new(cls, data, requires_grad: bool = False): return cls(data, requires_grad)

    @classmethod
    def from_tensor(cls, t): return cls(t, False)

    # ---- accessors
    def data(self): return self.tensor.detach()
    def shape(self): return tuple(self.tensor.shape)
    def numel(self): return self.tensor.numel()
    def requires_grad(self): return self.tensor.requires_grad
    def is_leaf(self): return self.tensor.is_leaf
    def grad(self): return self.tensor.grad
    def grad_fn(self): return self.tensor.grad_fn
    def zero_grad(self): self.tensor.grad = None
    def detach(self): return Variable(self.tensor.detach())
    def item(self): return self.tensor.item()
    def to_vec(self): return self.tensor.detach().flatten().tolist()

    def backward(self, grad=None):
        if grad is None and self.tensor.numel() != 1:
            grad = torch.ones_like(self.tensor)
        self.tensor.backward(grad.tensor if isinstance(grad, Variable) else grad)

    # ---- ops
    def _w(self, t): return Variable(t)
    def _u(self, o): return o.tensor if isinstance(o, Variable) else o
    def add_var(self, o): return self._w(self.tensor + self._u(o))
    def sub_var(self, o): return self._w(self.tensor - self._u(o))
    def mul_var(self, o): return self._w(self.tensor * self._u(o))
    def div_var(self, o): return self._w(self.tensor / self._u(o))
    def add_scalar(self, s): return self._w(self.tensor + s)
    def mul_scalar(self, s): return self._w(self.tensor * s)
    def neg_var(self): return self._w(-self.tensor)
    def matmul(self, o): return self._w(self.tensor @ self._u(o))
    def pow(self, e): return self._w(self.tensor.pow(e))
    def sqrt(self): return self._w(self.tensor.sqrt())
    def exp(self): return self._w(self.tensor.exp())
    def log(self): return self._w(self.tensor.log())
    def relu(self): return self._w(torch.relu(self.tensor))
    def sigmoid(self): return self._w(torch.sigmoid(self.tensor))
    def tanh(self): return self._w(torch.tanh(self.tensor))
    def gelu(self): return self._w(F.gelu(self.tensor, approximate="tanh"))
    def silu(self): return self._w(F.silu(self.tensor))
    def softmax(self, dim=-1): return self._w(torch.softmax(self.tensor, dim))
    def log_softmax(self, dim=-1): return self._w(torch.log_softmax(self.tensor, dim))
    def sum(self): return self._w(self.tensor.sum())
    def mean(self): return self._w(self.tensor.mean())
    def mean_dim(self, dim, keepdim=False): return self._w(self.tensor.mean(dim, keepdim))
    def var_dim(self, dim, keepdim=False): return self._w(self.tensor.var(dim, unbiased=False, keepdim=keepdim))
    def reshape(self, *shape): return self._w(self.tensor.reshape(*shape))
    def transpose(self, a, b): return self._w(self.tensor.transpose(a, b))
    def narrow(self, dim, start, length): return self._w(self.tensor.narrow(dim, start, length))
    def slice(self, ranges): return self._w(self.tensor[tuple(slice(a, b) for a, b in ranges)])
    def expand(self, *shape): return self._w(self.tensor.expand(*shape))
    def mse_loss(self, target): return self._w(F.mse_loss(self.tensor, self._u(target)))
    def binary_cross_entropy(self, target): return self._w(F.binary_cross_entropy(self.tensor, self._u(target)))
    def sub_scalar(self, s): return self._w(self.tensor - s)
    def div_scalar(self, s): return self._w(self.tensor / s)
    # operator forms under the reference's short names
    def add(self, o): return self.add_var(o)
    def sub(self, o): return self.sub_var(o)
    def mul(self, o): return self.mul_var(o)
    def div(self, o): return self.div_var(o)
    def ndim(self) -> int: return self.tensor.dim()

    @classmethod
    def from_tensor_with_grad(cls, t, requires_grad: bool = True): return cls(t, requires_grad)

    def clone_var(self):
        """A new leaf with a copy of the data and the same ``requires_grad``."""
        return Variable(self.tensor.detach().clone(), self.tensor.requires_grad)

    def requires_grad_(self, flag: bool = True):
        self.tensor.requires_grad_(flag)
        return self

    def set_grad(self, grad) -> None:
        self.tensor.grad = None if grad is None else torch.as_tensor(grad, dtype=self.tensor.dtype).reshape(self.tensor.shape).clone()

    def accumulate_grad(self, grad) -> None:
        """Adds ``grad`` to the stored gradient (sets it when there is none)."""
        g = torch.as_tensor(grad, dtype=self.tensor.dtype).reshape(self.tensor.shape)
        self.tensor.grad = g.clone() if self.tensor.grad is None else self.tensor.grad + g

    __add__ = add_var
    __sub__ = sub_var
    __mul__ = mul_var
    __truediv__ = div_var
    __neg__ = neg_var
    __matmul__ = matmul

    def __repr__(self): return f"Variable({self.tensor!r})"


def backward(output, grad=None) -> None:
    """Free-function form (crates/axonml-autograd/src/backward.rs:28)."""
    (output if isinstance(output, Variable) else Variable(output)).backward(grad)


def numerical_gradient(f, x: torch.Tensor, eps: float = 1e-4) -> torch.Tensor:
    """Central-difference gradient of a scalar function (backward.rs:117)."""
    x = x.detach().clone().double()
    g = torch.zeros_like(x)
    flat, gf = x.view(-1), g.view(-1)
    for i in range(flat.numel()):
        old = flat[i].item()
        flat[i] = old + eps
        hi = float(f(x.clone()))
        flat[i] = old - eps
        lo = float(f(x.clone()))
        flat[i] = old
        gf[i] = (hi - lo) / (2 * eps)
    return g


def gradcheck(f, x: torch.Tensor, rtol: float = 1e-3, atol: float = 1e-4, eps: float = 1e-4) -> bool:
    """Compares autograd with the numerical gradient (backward.rs:159)."""
    xa = x.detach().clone().double().requires_grad_(True)
    out = f(xa)
    out = out.tensor if isinstance(out, Variable) else out
    out.backward()
    num = numerical_gradient(lambda t: (lambda o: o.tensor if isinstance(o, Variable) else o)(f(t)).item(), x, eps)
    return bool(torch.allclose(xa.grad, num, rtol=rtol, atol=atol))
