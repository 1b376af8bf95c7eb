"""Tensor facade (crates/axonml-tensor): ``Tensor`` is ``torch.Tensor``; creation functions, views,
operations and sparse formats keep the reference's names."""
import torch

from ..core import DType, Device, Error
from . import ops, shape, sparse, view
from .creation import (arange, diag, empty, eye, from_vec, full, full_like, linspace, logspace, normal,
                       ones, ones_like, rand, randint, randn, scalar, uniform, zeros, zeros_like)
from .shape import Shape, Strides
from .sparse import SparseCOO, SparseCSR, SparseFormat, SparseTensor
from .view import SliceSpec, slice_with

Tensor = torch.Tensor
