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
