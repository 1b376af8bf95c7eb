"""Functional API (crates/axonml-nn/src/functional.rs:17-296)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import elementwise as E
from ..ops import loss as L
from ..ops import norm as Nm
from ..ops.linear import linear as _linear
from . import activation as A


def relu(x): return A._act(x, "relu")
def leaky_relu(x, negative_slope: float = 0.01): return A._act(x, "leaky_relu", negative_slope)
def sigmoid(x): return A._act(x, "sigmoid")
def tanh(x): return A._act(x, "tanh")
def gelu(x): return A._act(x, "gelu")
def silu(x): return A._act(x, "silu")
def elu(x, alpha: float = 1.0): return A._act(x, "elu", alpha)
def softmax(x, dim: int = -1): return L.softmax(x, dim)
def log_softmax(x, dim: int = -1): return L.log_softmax(x, dim)
def linear(x, weight, bias=None): return _linear(x, weight, bias)


def layer_norm(x, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    if weight is not None and len(normalized_shape) == 1:
        return Nm.layer_norm(x, weight, bias, eps)
    return F.layer_norm(x, tuple(normalized_shape), weight, bias, eps)


def dropout(x, p: float = 0.5, training: bool = True): return E.dropout(x, p, training)
def mse_loss(input, target): return F.mse_loss(input, target)
def cross_entropy(input, target): return L.cross_entropy(input, target.long() if target.is_floating_point() else target)
def binary_cross_entropy(input, target): return F.binary_cross_entropy(input, target)
def adaptive_avg_pool2d(x, output_size):
    from ..ops.pool import adaptive_avg_pool2d as _aap
    return _aap(x, output_size)
