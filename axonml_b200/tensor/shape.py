"""Shape and stride arithmetic.

Parity: crates/axonml-tensor/src/shape.rs:26-395 (``Shape`` / ``Strides`` aliases, ``numel``,
``contiguous_strides`` (row-major), ``is_contiguous``, ``linear_index``, ``unravel_index``,
``broadcast_shape`` / ``broadcast_strides`` / ``can_broadcast`` with NumPy rules, ``reshape`` with
one inferred ``-1``, ``squeeze`` / ``unsqueeze``, ``transpose_shape`` / ``transpose_strides``,
``normalize_dim``, ``validate_indices``).  Shapes and strides are tuples of ints, strides in
elements; the functions raise the framework's error classes."""
from __future__ import annotations

from ..core.error import BroadcastError, IndexOutOfBounds, InvalidDimension, InvalidOperation, ShapeMismatch

Shape = tuple      # of non-negative ints
Strides = tuple    # of ints, in elements (a broadcast dimension has stride 0)


def numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def contiguous_strides(shape) -> Strides:
    out, acc = [], 1
    for d in reversed(tuple(shape)):
        out.append(acc)
        acc *= int(d)
    return tuple(reversed(out))


def is_contiguous(shape, strides) -> bool:
    """Row-major and dense; dimensions of extent 1 may carry any stride, an empty tensor is contiguous."""
    if numel(shape) == 0:
        return True
    expected = 1
    for d, s in zip(reversed(tuple(shape)), reversed(tuple(strides))):
        if d != 1 and s != expected:
            return False
        expected *= d
    return True


def linear_index(indices, strides) -> int:
    return sum(int(i) * int(s) for i, s in zip(indices, strides))


def unravel_index(linear: int, shape) -> list:
    out = []
    for d in reversed(tuple(shape)):
        out.append(linear % d if d else 0)
        linear = linear // d if d else 0
    return list(reversed(out))


def broadcast_shape(shape1, shape2) -> Shape:
    a, b = tuple(shape1), tuple(shape2)
    out = []
    for i in range(max(len(a), len(b))):
        x = a[len(a) - 1 - i] if i < len(a) else 1
        y = b[len(b) - 1 - i] if i < len(b) else 1
        if x == y or y == 1:
            out.append(x)
        elif x == 1:
            out.append(y)
        else:
            raise BroadcastError(a, b)
    return tuple(reversed(out))


def can_broadcast(shape1, shape2) -> bool:
    try:
        broadcast_shape(shape1, shape2)
        return True
    except BroadcastError:
        return False


def broadcast_strides(shape, strides, target_shape) -> Strides:
    """Strides that view a tensor of ``shape`` as ``target_shape``: 0 where a dimension is
    stretched or added in front."""
    shape, strides, target = tuple(shape), tuple(strides), tuple(target_shape)
    if len(shape) > len(target):
        raise BroadcastError(shape, target)
    lead = len(target) - len(shape)
    out = [0] * lead
    for d, s, t in zip(shape, strides, target[lead:]):
        if d == t:
            out.append(s)
        elif d == 1:
            out.append(0)
        else:
            raise BroadcastError(shape, target)
    return tuple(out)


def reshape(old_shape, new_shape) -> Shape:
    old_n = numel(old_shape)
    out, infer, known = [], None, 1
    for i, d in enumerate(new_shape):
        d = int(d)
        if d == -1:
            if infer is not None:
                raise InvalidOperation("Can only have one -1 in reshape")
            infer = i
            out.append(0)
        elif d < 0:
            raise InvalidOperation("Invalid dimension in reshape")
        else:
            known *= d
            out.append(d)
    if infer is not None:
        if known == 0 or old_n % known:
            raise InvalidOperation("Cannot infer dimension: not evenly divisible")
        out[infer] = old_n // known
    elif known != old_n:
        raise ShapeMismatch(tuple(old_shape), tuple(out))
    return tuple(out)


def squeeze(shape, dim: int | None = None) -> Shape:
    shape = tuple(shape)
    if dim is None:
        return tuple(d for d in shape if d != 1)
    if 0 <= dim < len(shape) and shape[dim] == 1:
        return shape[:dim] + shape[dim + 1:]
    return shape


def unsqueeze(shape, dim: int) -> Shape:
    shape = tuple(shape)
    if not 0 <= dim <= len(shape):
        raise InvalidDimension(dim, len(shape) + 1)
    return shape[:dim] + (1,) + shape[dim:]


def _swap(seq, dim0: int, dim1: int) -> tuple:
    out = list(seq)
    out[dim0], out[dim1] = out[dim1], out[dim0]
    return tuple(out)


def transpose_shape(shape, dim0: int, dim1: int) -> Shape:
    n = len(tuple(shape))
    for d in (dim0, dim1):
        if not 0 <= d < n:
            raise InvalidDimension(d, n)
    return _swap(shape, dim0, dim1)


def transpose_strides(strides, dim0: int, dim1: int) -> Strides:
    return _swap(strides, dim0, dim1)


def normalize_dim(dim: int, ndim: int) -> int:
    d = dim + ndim if dim < 0 else dim
    if not 0 <= d < ndim:
        raise InvalidDimension(dim, ndim)
    return d


def validate_indices(indices, shape) -> None:
    indices, shape = tuple(indices), tuple(shape)
    if len(indices) != len(shape):
        raise InvalidOperation(f"Expected {len(shape)} indices, got {len(indices)}")
    for i, d in zip(indices, shape):
        if not 0 <= i < d:
            raise IndexOutOfBounds(i, d)
