"""Tensor facade (crates/axonml-tensor): ``Tensor`` is ``torch.Tensor``; creation functions, views,
operations and sparse formats keep the reference's names."""
import builtins as _builtins

import torch

from ..core import DType, Device, Error
from . import ops, shape, sparse, view
from .creation import (arange, diag, empty, eye, from_vec, full, full_like, linspace, logspace, normal,
                       ones, ones_like, rand, randint, randn, scalar, uniform, zeros, zeros_like)
from .shape import Shape, Strides
from .sparse import SparseCOO, SparseCSR, SparseFormat, SparseTensor
from .view import SliceSpec, slice_with

Tensor = torch.Tensor
_py_slice = _builtins.slice


# The reference's ``Tensor`` methods (crates/axonml-tensor/src/tensor.rs) that torch.Tensor spells
# differently, as functions of this module.
from .ops import add_scalar, gelu, ln, mean_dim, mul_scalar, silu, var_dim  # noqa: E402
from .view import slice_dim0  # noqa: E402


def from_storage(storage, shape):
    """Tensor over the elements of a ``core.Storage`` (a view when the storage is contiguous)."""
    return storage.as_tensor().reshape(tuple(shape))


def from_slice(data, shape, dtype=torch.float32, device=None):
    """Copy of a flat sequence in the given shape (tensor.rs: ``Tensor::from_slice``)."""
    return from_vec(list(data), shape, dtype=dtype, device=device)


def strides(t) -> list: return list(t.stride())
def is_empty(t) -> bool: return t.numel() == 0
def is_scalar(t) -> bool: return t.dim() == 0


def get(t, indices):
    """Python scalar at a multi-dimensional index; ``IndexError`` when out of range."""
    idx = tuple(indices)
    if len(idx) != t.dim():
        raise IndexError(f"{len(idx)} indices for a tensor of {t.dim()} dimensions")
    return t[idx].item()


def to_vec(t) -> list:
    """Elements in row-major order as a Python list."""
    return t.detach().reshape(-1).cpu().tolist()


def to_device(t, device):
    """Copy on ``device`` (a ``core.Device``, a torch device or a string)."""
    return t.to(device.to_torch() if hasattr(device, "to_torch") else device)


def clone_deep(t):
    """Copy with its own contiguous storage."""
    return t.detach().clone(memory_format=torch.contiguous_format)


def slice(t, ranges):  # noqa: A001 - the reference's method name
    """Sub-tensor over ``(start, end)`` pairs, one per leading dimension (tensor.rs: ``slice``)."""
    return t[tuple(_py_slice(a, b) for a, b in ranges)]
