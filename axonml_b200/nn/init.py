"""Initialisers with the reference's names and formulas (crates/axonml-nn/src/init.rs:17-267).
Each returns a new fp32 tensor; shapes follow the reference ([fan_out, fan_in] for 2-D)."""
from __future__ import annotations

import enum
import math

import torch


def zeros(*shape): return torch.zeros(*shape)
def ones(*shape): return torch.ones(*shape)
def constant(shape, value: float): return torch.full(tuple(shape), float(value))
def uniform(*shape): return torch.rand(*shape)
def uniform_range(shape, low: float, high: float): return torch.empty(tuple(shape)).uniform_(low, high)
def randn(*shape): return torch.randn(*shape)
def normal(shape, mean: float, std: float): return torch.empty(tuple(shape)).normal_(mean, std)


def xavier_uniform(fan_in: int, fan_out: int):
    a = math.sqrt(6.0 / (fan_in + fan_out))
    return torch.empty(fan_out, fan_in).uniform_(-a, a)


def xavier_normal(fan_in: int, fan_out: int):
    return torch.empty(fan_out, fan_in).normal_(0.0, math.sqrt(2.0 / (fan_in + fan_out)))


glorot_uniform = xavier_uniform
glorot_normal = xavier_normal


def kaiming_uniform(fan_out: int, fan_in: int):
    bound = math.sqrt(6.0 / fan_in)
    return torch.empty(fan_out, fan_in).uniform_(-bound, bound)


def kaiming_normal(fan_out: int, fan_in: int):
    return torch.empty(fan_out, fan_in).normal_(0.0, math.sqrt(2.0 / fan_in))


he_uniform = kaiming_uniform
he_normal = kaiming_normal


def orthogonal(rows: int, cols: int, gain: float = 1.0):
    t = torch.empty(rows, cols)
    torch.nn.init.orthogonal_(t, gain)
    return t


def sparse(rows: int, cols: int, sparsity: float, std: float = 0.01):
    t = torch.empty(rows, cols).normal_(0.0, std)
    t[torch.rand(rows, cols) < sparsity] = 0.0
    return t


def eye(n: int): return torch.eye(n)
def diag(values): return torch.diag(torch.as_tensor(values, dtype=torch.float32))


class InitMode(enum.Enum):
    Zeros = "zeros"
    Ones = "ones"
    Constant = "constant"
    Uniform = "uniform"
    Normal = "normal"
    XavierUniform = "xavier_uniform"
    XavierNormal = "xavier_normal"
    KaimingUniform = "kaiming_uniform"
    KaimingNormal = "kaiming_normal"
    Orthogonal = "orthogonal"

    def init(self, shape, value: float = 0.0):
        shape = tuple(shape)
        fan_out = shape[0] if shape else 1
        fan_in = int(torch.tensor(shape[1:]).prod().item()) if len(shape) > 1 else fan_out
        if self is InitMode.Zeros: return torch.zeros(shape)
        if self is InitMode.Ones: return torch.ones(shape)
        if self is InitMode.Constant: return torch.full(shape, value)
        if self is InitMode.Uniform: return torch.rand(shape)
        if self is InitMode.Normal: return torch.randn(shape)
        if self is InitMode.XavierUniform: return xavier_uniform(fan_in, fan_out).reshape(shape)
        if self is InitMode.XavierNormal: return xavier_normal(fan_in, fan_out).reshape(shape)
        if self is InitMode.KaimingUniform: return kaiming_uniform(fan_out, fan_in).reshape(shape)
        if self is InitMode.KaimingNormal: return kaiming_normal(fan_out, fan_in).reshape(shape)
        return orthogonal(fan_out, fan_in).reshape(shape)
