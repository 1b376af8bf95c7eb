"""Automatic mixed precision (crates/axonml-autograd/src/amp.rs).  ``autocast(dtype)`` is a real
context manager: inside it the matmul-class ops (Linear, conv, attention) compute in ``dtype``
(bf16 by default) while norms, softmax and losses keep fp32 statistics."""
from __future__ import annotations

import contextlib
import enum

import torch

from ..core.dtype import as_torch_dtype


class AutocastPolicy(enum.Enum):
    LowerPrecision = "lower"      # matmul-class ops
    FullPrecision = "full"        # reductions, norms, losses
    Promote = "promote"           # mixed inputs take the widest type


def _device_type() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


@contextlib.contextmanager
def autocast(dtype=torch.bfloat16, enabled: bool = True, device_type: str | None = None):
    with torch.autocast(device_type or _device_type(), dtype=as_torch_dtype(dtype), enabled=enabled):
        yield


@contextlib.contextmanager
def disable_autocast(device_type: str | None = None):
    with torch.autocast(device_type or _device_type(), enabled=False):
        yield


AutocastGuard = autocast


def is_autocast_enabled(device_type: str | None = None) -> bool:
    return torch.is_autocast_enabled(device_type or _device_type())
