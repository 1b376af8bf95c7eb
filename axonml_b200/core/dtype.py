"""Runtime dtype enum.  Mirrors crates/axonml-core/src/dtype.rs:28-52 and adds BF16, which the
reference lacks and every GPU configuration here computes in."""
from __future__ import annotations

import enum

import torch


class DType(enum.Enum):
    F16 = "f16"
    BF16 = "bf16"
    F32 = "f32"
    F64 = "f64"
    I8 = "i8"
    I16 = "i16"
    I32 = "i32"
    I64 = "i64"
    U8 = "u8"
    U32 = "u32"
    U64 = "u64"
    Bool = "bool"

    # ---- reference API (dtype.rs:54-130)
    def size_of(self) -> int:
        return _SIZES[self]

    def is_float(self) -> bool:
        return self in (DType.F16, DType.BF16, DType.F32, DType.F64)

    def is_signed(self) -> bool:
        return self.is_float() or self in (DType.I8, DType.I16, DType.I32, DType.I64)

    def is_integer(self) -> bool:
        return self in (DType.I8, DType.I16, DType.I32, DType.I64, DType.U8, DType.U32, DType.U64)

    def name_str(self) -> str:
        return self.value

    def default_float() -> "DType":  # type: ignore[misc]
        return DType.F32

    def default_int() -> "DType":  # type: ignore[misc]
        return DType.I64

    # ---- torch interop
    def to_torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        return _FROM_TORCH[dt]

    def __str__(self) -> str:
        return self.value


_SIZES = {DType.F16: 2, DType.BF16: 2, DType.F32: 4, DType.F64: 8, DType.I8: 1, DType.I16: 2,
          DType.I32: 4, DType.I64: 8, DType.U8: 1, DType.U32: 4, DType.U64: 8, DType.Bool: 1}
_TO_TORCH = {DType.F16: torch.float16, DType.BF16: torch.bfloat16, DType.F32: torch.float32,
             DType.F64: torch.float64, DType.I8: torch.int8, DType.I16: torch.int16,
             DType.I32: torch.int32, DType.I64: torch.int64, DType.U8: torch.uint8,
             DType.U32: torch.uint32, DType.U64: torch.uint64, DType.Bool: torch.bool}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


def as_torch_dtype(dt) -> torch.dtype:
    if isinstance(dt, torch.dtype):
        return dt
    if isinstance(dt, DType):
        return dt.to_torch()
    if isinstance(dt, str):
        return DType(dt).to_torch()
    raise TypeError(f"not a dtype: {dt!r}")


# ---------------------------------------------------------------------------------------------
# Scalar tower (dtype.rs:134-256).  The reference's traits are implemented per Rust scalar type;
# here one descriptor object per dtype carries the same associated constants, and the classes
# answer "does this dtype belong to the group" the way a trait bound would.
class Scalar:
    """Any element type a tensor can hold.  ``Scalar.of(dtype)`` returns the descriptor."""
    _accepts = staticmethod(lambda d: True)

    def __init__(self, dtype: DType):
        self.DTYPE = dtype

    def dtype(self) -> DType:
        return self.DTYPE

    @classmethod
    def accepts(cls, dt) -> bool:
        d = dt if isinstance(dt, DType) else DType.from_torch(as_torch_dtype(dt))
        return cls._accepts(d)

    @classmethod
    def of(cls, dt):
        d = dt if isinstance(dt, DType) else DType.from_torch(as_torch_dtype(dt))
        if not cls._accepts(d):
            raise TypeError(f"{d} is not a {cls.__name__} type")
        return cls(d)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.DTYPE})"


class Numeric(Scalar):
    """Scalars with arithmetic and an order: every dtype but Bool."""
    _accepts = staticmethod(lambda d: d is not DType.Bool)

    def __init__(self, dtype: DType):
        super().__init__(dtype)
        t = dtype.to_torch()
        info = torch.finfo(t) if dtype.is_float() else torch.iinfo(t)
        cast = float if dtype.is_float() else int
        self.ZERO, self.ONE = cast(0), cast(1)
        self._min, self._max = cast(info.min), cast(info.max)

    def min_value(self): return self._min
    def max_value(self): return self._max


class Float(Numeric):
    """Floating-point scalars: F16, BF16, F32, F64."""
    _accepts = staticmethod(lambda d: d.is_float())

    def __init__(self, dtype: DType):
        super().__init__(dtype)
        info = torch.finfo(dtype.to_torch())
        self.NAN, self.INFINITY, self.NEG_INFINITY = float("nan"), float("inf"), float("-inf")
        self.EPSILON, self.MIN_POSITIVE = float(info.eps), float(info.tiny)
