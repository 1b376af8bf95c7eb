"""Tensor operations (crates/axonml-tensor/src/ops/mod.rs:73-780, tensor.rs:900-1081).  Elementwise
and activation ops on CUDA fp32/bf16 tensors run the hand-written kernels; ``softmax`` /
``log_softmax`` are dim-aware and numerically stable (the reference normalises over the whole
tensor and computes ``ln(softmax)``)."""
from __future__ import annotations

import torch

from ..ops import elementwise as E
from ..ops import loss as L
from ..ops.gemm import gemm_bf16, gemm_supported


def _same(a, b):
    return torch.is_tensor(b) and a.shape == b.shape and a.dtype == b.dtype


def add(a, b): return E.binary(a, b, "add") if _same(a, b) else a + b
def sub(a, b): return E.binary(a, b, "sub") if _same(a, b) else a - b
def mul(a, b): return E.binary(a, b, "mul") if _same(a, b) else a * b
def div(a, b): return E.binary(a, b, "div") if _same(a, b) else a / b
def add_scalar(a, s): return E.unary(a, "add_scalar", float(s))
def mul_scalar(a, s): return E.unary(a, "scale", float(s))
def neg(a): return E.unary(a, "neg")
def abs(a): return E.unary(a, "abs")  # noqa: A001
def sqrt(a): return E.unary(a, "sqrt")
def exp(a): return E.unary(a, "exp")
def ln(a): return E.unary(a, "log")
def log(a): return E.unary(a, "log")
def square(a): return E.unary(a, "square")
def pow(a, e): return E.unary(a, "pow_scalar", float(e)) if not torch.is_tensor(e) else E.binary(a, e, "pow")  # noqa: A001
def relu(a): return E.unary(a, "relu")
def sigmoid(a): return E.unary(a, "sigmoid")
def tanh(a): return E.unary(a, "tanh")
def gelu(a): return E.unary(a, "gelu")
def silu(a): return E.unary(a, "silu")
def elu(a, alpha=1.0): return E.unary(a, "elu", float(alpha))
def leaky_relu(a, slope=0.01): return E.unary(a, "leaky_relu", float(slope))
def clamp(a, lo, hi): return E.unary(a, "clamp", float(lo), float(hi))
def clamp_min(a, lo): return torch.clamp_min(a, lo)
def clamp_max(a, hi): return torch.clamp_max(a, hi)
def softmax(a, dim=-1): return L.softmax(a, dim)
def log_softmax(a, dim=-1): return L.log_softmax(a, dim)
def where_cond(cond, a, b): return torch.where(cond, a, b)
def eq(a, b): return a == b
def lt(a, b): return a < b
def gt(a, b): return a > b


def matmul(a, b):
    """2-D and equal-batch N-D matrix product (tensor.rs:1020-1081); bf16 2-D products on a B200
    use the tcgen05 kernel."""
    if a.dim() == 2 and b.dim() == 2 and gemm_supported(a, b) and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0:
        return gemm_bf16(a, b, trans_b=False)
    return torch.matmul(a, b)


def dot(a, b): return torch.dot(a.flatten(), b.flatten())
def sum(a, dim=None, keepdim=False): return a.sum() if dim is None else a.sum(dim, keepdim)  # noqa: A001
def prod(a): return a.prod()
def mean(a): return a.mean()
def mean_dim(a, dim, keepdim=False): return a.mean(dim, keepdim)
def var_dim(a, dim, keepdim=False): return a.var(dim, unbiased=False, keepdim=keepdim)
def max(a): return a.max()  # noqa: A001
def min(a): return a.min()  # noqa: A001
def argmax(a, dim=None): return a.argmax(dim)
def argmin(a, dim=None): return a.argmin(dim)
def topk(a, k, dim=-1, largest=True): return torch.topk(a, k, dim, largest)
def sort(a, dim=-1, descending=False): return torch.sort(a, dim, descending)
def argsort(a, dim=-1, descending=False): return torch.argsort(a, dim, descending)
def scatter(a, dim, index, src): return a.scatter(dim, index, src)
def gather(a, dim, index): return a.gather(dim, index)
def masked_select(a, mask): return a.masked_select(mask)
def masked_fill(a, mask, value): return a.masked_fill(mask, value)
def nonzero(a): return a.nonzero()
def unique(a): return a.unique()
def flip(a, dims): return a.flip(dims)
def roll(a, shifts, dims): return a.roll(shifts, dims)
def cat(tensors, dim=0): return torch.cat(list(tensors), dim)
def stack(tensors, dim=0): return torch.stack(list(tensors), dim)
