"""Views and shape helpers (crates/axonml-tensor/src/view.rs:98-409, shape.rs:26-376)."""
from __future__ import annotations

import torch

from ..core.error import BroadcastError, InvalidDimension, ShapeMismatch


def reshape(t, shape): return t.reshape(tuple(shape))
def flatten(t, start=0, end=-1): return t.flatten(start, end)
def squeeze(t, dim=None): return t.squeeze() if dim is None else t.squeeze(dim)
def unsqueeze(t, dim): return t.unsqueeze(dim)
def transpose(t, a, b): return t.transpose(a, b)
def t(x): return x.t()
def permute(t, dims): return t.permute(tuple(dims))
def contiguous(t): return t.contiguous()
def slice_dim0(t, start, end): return t[start:end]
def select(t, dim, index): return t.select(dim, index)
def narrow(t, dim, start, length): return t.narrow(dim, start, length)
def chunk(t, n, dim=0): return list(t.chunk(n, dim))
def split(t, size, dim=0): return list(t.split(size, dim))
def expand(t, shape): return t.expand(tuple(shape))


def numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def contiguous_strides(shape) -> list:
    st, acc = [], 1
    for s in reversed(list(shape)):
        st.append(acc)
        acc *= s
    return list(reversed(st))


def is_contiguous(shape, strides) -> bool:
    return list(strides) == contiguous_strides(shape)


def normalize_dim(dim: int, ndim: int) -> int:
    if not -ndim <= dim < ndim:
        raise InvalidDimension(dim, ndim)
    return dim % ndim


def broadcast_shape(a, b) -> list:
    out = []
    for x, y in zip(reversed([1] * (len(b) - len(a)) + list(a)), reversed([1] * (len(a) - len(b)) + list(b))):
        if x != y and x != 1 and y != 1:
            raise BroadcastError(a, b)
        out.append(x if y == 1 else y)
    return list(reversed(out))


def broadcast_strides(shape, strides, target) -> list:
    pad = len(target) - len(shape)
    out = [0] * pad
    for s, st, tgt in zip(shape, strides, target[pad:]):
        out.append(0 if (s == 1 and tgt != 1) else st)
    return out


def reshape_infer(shape, new_shape) -> list:
    total = numel(shape)
    new = list(new_shape)
    if new.count(-1) > 1:
        raise ShapeMismatch(shape, new_shape)
    if -1 in new:
        known = numel([s for s in new if s != -1])
        if known == 0 or total % known:
            raise ShapeMismatch(shape, new_shape)
        new[new.index(-1)] = total // known
    if numel(new) != total:
        raise ShapeMismatch(shape, new_shape)
    return new


def linear_index(indices, strides) -> int:
    return sum(i * s for i, s in zip(indices, strides))


def unravel_index(index: int, shape) -> list:
    out = []
    for s in reversed(list(shape)):
        out.append(index % s)
        index //= s
    return list(reversed(out))


class SliceSpec:
    """One entry of a multi-dimensional index (view.rs:27-85): ``SliceSpec.Index(i)`` picks one
    position and drops the dimension, ``SliceSpec.range(a, b)`` / ``range_step(a, b, s)`` /
    ``from_(a)`` / ``to(b)`` take a strided range, ``SliceSpec.All`` keeps the dimension and
    ``SliceSpec.NewAxis`` inserts one of extent 1.  Negative positions count from the end."""

    def __init__(self, kind: str, start=None, stop=None, step: int = 1):
        self.kind, self.start, self.stop, self.step = kind, start, stop, step

    @classmethod
    def Index(cls, i: int): return cls("index", int(i))
    @classmethod
    def Range(cls, start=None, stop=None, step: int = 1): return cls("range", start, stop, step)
    @classmethod
    def range(cls, start: int, stop: int): return cls("range", start, stop, 1)
    @classmethod
    def range_step(cls, start: int, stop: int, step: int): return cls("range", start, stop, step)
    @classmethod
    def from_(cls, start: int): return cls("range", start, None, 1)
    @classmethod
    def to(cls, stop: int): return cls("range", None, stop, 1)

    def as_index(self):
        """The Python indexing object that means the same."""
        if self.kind == "index":
            return self.start
        if self.kind == "range":
            return slice(self.start, self.stop, self.step)
        return slice(None) if self.kind == "all" else None

    def __repr__(self) -> str:
        return {"index": f"Index({self.start})", "range": f"Range({self.start}, {self.stop}, {self.step})", "all": "All",
                "newaxis": "NewAxis"}[self.kind]


SliceSpec.All = SliceSpec("all")
SliceSpec.NewAxis = SliceSpec("newaxis")


def slice_with(t, specs):
    """View of ``t`` selected by a list of ``SliceSpec`` (fewer specs than dimensions leave the
    rest whole).  Steps must be positive: a view cannot run backwards through storage here."""
    from ..core.error import InvalidOperation
    specs = list(specs)
    if sum(s.kind != "newaxis" for s in specs) > t.dim():
        raise InvalidOperation(f"{len(specs)} index entries for a tensor with {t.dim()} dimensions")
    if any(s.kind == "range" and s.step <= 0 for s in specs):
        raise InvalidOperation("slice step must be positive")
    return t[tuple(s.as_index() for s in specs)]
