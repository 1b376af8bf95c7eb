"""Tensor creation functions (crates/axonml-tensor/src/creation.rs:38-287)."""
from __future__ import annotations

import torch

from ..core.device import as_torch_device
from ..core.dtype import as_torch_dtype


def _kw(dtype=None, device=None):
    kw = {}
    if dtype is not None:
        kw["dtype"] = as_torch_dtype(dtype)
    if device is not None:
        kw["device"] = as_torch_device(device)
    return kw


def zeros(*shape, dtype=None, device=None): return torch.zeros(*shape, **_kw(dtype, device))
def ones(*shape, dtype=None, device=None): return torch.ones(*shape, **_kw(dtype, device))
def full(shape, value, dtype=None, device=None): return torch.full(tuple(shape), value, **_kw(dtype, device))
def empty(*shape, dtype=None, device=None): return torch.empty(*shape, **_kw(dtype, device))
def zeros_like(t): return torch.zeros_like(t)
def ones_like(t): return torch.ones_like(t)
def full_like(t, value): return torch.full_like(t, value)
def eye(n, dtype=None, device=None): return torch.eye(n, **_kw(dtype, device))
def diag(values): return torch.diag(torch.as_tensor(values))
def rand(*shape, dtype=None, device=None): return torch.rand(*shape, **_kw(dtype, device))
def randn(*shape, dtype=None, device=None): return torch.randn(*shape, **_kw(dtype, device))
def uniform(shape, low=0.0, high=1.0, device=None): return torch.empty(tuple(shape), **_kw(None, device)).uniform_(low, high)
def normal(shape, mean=0.0, std=1.0, device=None): return torch.empty(tuple(shape), **_kw(None, device)).normal_(mean, std)
def randint(low, high, shape, device=None): return torch.randint(low, high, tuple(shape), **_kw(None, device))
def arange(start, end=None, step=1, dtype=None, device=None):
    if end is None:
        start, end = 0, start
    return torch.arange(start, end, step, **_kw(dtype, device))
def linspace(start, end, steps, device=None): return torch.linspace(start, end, steps, **_kw(None, device))
def logspace(start, end, steps, base=10.0, device=None): return torch.logspace(start, end, steps, base=base, **_kw(None, device))
def from_vec(data, shape=None, dtype=None, device=None):
    t = torch.tensor(data, **_kw(dtype or torch.float32, device))
    return t.reshape(shape) if shape is not None else t
def scalar(value, dtype=None, device=None): return torch.tensor(value, **_kw(dtype or torch.float32, device))
