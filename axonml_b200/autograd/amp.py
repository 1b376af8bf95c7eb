"""Automatic mixed precision (crates/axonml-autograd/src/amp.rs).  ``autocast(dtype)`` is a real
context manager: inside it the matmul-class ops (Linear, conv, attention) compute in ``dtype``
(bf16 by default) while norms, softmax and losses keep fp32 statistics."""
from __future__ import annotations

import contextlib
import enum
import threading

import torch

from ..core.dtype import as_torch_dtype


class AutocastPolicy(enum.Enum):
    LowerPrecision = "lower"      # matmul-class ops
    FullPrecision = "full"        # reductions, norms, losses
    Promote = "promote"           # mixed inputs take the widest type


def _device_type() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


_TLS = threading.local()    # .stack: dtypes of the enabled autocast regions this thread is inside


def _stack() -> list:
    st = getattr(_TLS, "stack", None)
    if st is None:
        st = _TLS.stack = []
    return st


@contextlib.contextmanager
def autocast(dtype=torch.bfloat16, enabled: bool = True, device_type: str | None = None):
    td = as_torch_dtype(dtype)
    with torch.autocast(device_type or _device_type(), dtype=td, enabled=enabled):
        if enabled:
            _stack().append(td)
        try:
            yield
        finally:
            if enabled:
                _stack().pop()


def autocast_dtype(device_type: str | None = None):
    """Compute dtype of the innermost autocast region as a ``DType`` (meaningful only while
    ``is_autocast_enabled()``; amp.rs:49-54)."""
    from ..core.dtype import DType
    if _stack():
        return DType.from_torch(_stack()[-1])
    return DType.from_torch(torch.get_autocast_dtype(device_type or _device_type()))


def autocast_depth() -> int:
    """How many enabled ``autocast`` regions are open (amp.rs:56-60)."""
    return len(_stack())


@contextlib.contextmanager
def disable_autocast(device_type: str | None = None):
    with torch.autocast(device_type or _device_type(), enabled=False):
        yield


AutocastGuard = autocast


def is_autocast_enabled(device_type: str | None = None) -> bool:
    return torch.is_autocast_enabled(device_type or _device_type())
