"""Quantisation types (crates/axonml-quant/src/types.rs:17-340): ``QuantType`` with block size,
bytes per block, bits per value and compression ratio; ``QuantizedTensor`` holding the packed
blocks.  Q5_0 / Q5_1 are real codecs and Q4_K is added (the reference maps Q5 to Q4_0 and has no
K-quants)."""
from __future__ import annotations

import dataclasses
import enum

import torch


class QuantError(Exception):
    pass


class QuantType(enum.Enum):
    Q8_0 = "q8_0"
    Q4_0 = "q4_0"
    Q4_1 = "q4_1"
    Q5_0 = "q5_0"
    Q5_1 = "q5_1"
    Q4_K = "q4_k"
    F16 = "f16"
    BF16 = "bf16"
    F32 = "f32"

    def block_size(self) -> int:
        return {QuantType.Q4_K: 256, QuantType.F16: 1, QuantType.BF16: 1, QuantType.F32: 1}.get(self, 32)

    def bytes_per_block(self) -> int:
        return {QuantType.Q8_0: 34, QuantType.Q4_0: 18, QuantType.Q4_1: 20, QuantType.Q5_0: 22,
                QuantType.Q5_1: 24, QuantType.Q4_K: 144, QuantType.F16: 2, QuantType.BF16: 2,
                QuantType.F32: 4}[self]

    def bits_per_value(self) -> float:
        return 8.0 * self.bytes_per_block() / self.block_size()

    def nominal_bits(self) -> int:
        return {QuantType.Q8_0: 8, QuantType.Q4_0: 4, QuantType.Q4_1: 4, QuantType.Q5_0: 5, QuantType.Q5_1: 5,
                QuantType.Q4_K: 4, QuantType.F16: 16, QuantType.BF16: 16, QuantType.F32: 32}[self]

    def compression_ratio(self) -> float:
        return 32.0 / self.nominal_bits()

    def is_block_quantized(self) -> bool:
        return self not in (QuantType.F16, QuantType.BF16, QuantType.F32)

    def codec_id(self) -> int:
        return {QuantType.Q8_0: 0, QuantType.Q4_0: 1, QuantType.Q4_1: 2, QuantType.Q5_0: 3,
                QuantType.Q5_1: 4, QuantType.Q4_K: 5}[self]

    def ggml_type(self) -> int:
        return {QuantType.F32: 0, QuantType.F16: 1, QuantType.Q4_0: 2, QuantType.Q4_1: 3, QuantType.Q5_0: 6,
                QuantType.Q5_1: 7, QuantType.Q8_0: 8, QuantType.Q4_K: 12, QuantType.BF16: 30}[self]

    @staticmethod
    def from_ggml_type(t: int) -> "QuantType":
        for q in QuantType:
            if q.ggml_type() == t:
                return q
        raise QuantError(f"unsupported GGML tensor type {t}")

    @staticmethod
    def from_str(s: str):
        s = s.strip().lower().replace("-", "_")
        alias = {"q8": "q8_0", "int8": "q8_0", "q4": "q4_0", "int4": "q4_0", "q5": "q5_0", "fp16": "f16",
                 "half": "f16", "fp32": "f32", "float": "f32", "q4k": "q4_k", "q4_k_m": "q4_k"}
        s = alias.get(s, s)
        for q in QuantType:
            if q.value == s:
                return q
        return None


@dataclasses.dataclass
class QuantizedTensor:
    shape: list
    quant_type: QuantType
    data: torch.Tensor            # uint8, packed blocks in row order
    layout: str = "ggml"          # "ggml" or "adjacent" (the reference's nibble order, Q4 only)

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def size_bytes(self) -> int: return self.data.numel()
    def num_blocks(self) -> int: return self.data.numel() // self.quant_type.bytes_per_block()
    def compression_ratio(self) -> float: return 4.0 * self.numel() / max(1, self.size_bytes())

    def to(self, device) -> "QuantizedTensor":
        return QuantizedTensor(self.shape, self.quant_type, self.data.to(device), self.layout)

    def block(self, index: int) -> "QuantizedBlock":
        """One block of the tensor as a ``QuantizedBlock`` (a copy of its bytes)."""
        n = self.quant_type.bytes_per_block()
        if not 0 <= index < self.num_blocks():
            raise IndexError(f"block {index} of {self.num_blocks()}")
        return QuantizedBlock(self.quant_type, bytes(self.data[index * n:(index + 1) * n].cpu().numpy().tobytes()), self.layout)

    def blocks(self):
        return (self.block(i) for i in range(self.num_blocks()))


@dataclasses.dataclass(frozen=True)
class QuantizedBlock:
    """One block of quantised values with its header (types.rs:128-288: ``Q8Block{scale: f16, data:
    [i8; 32]}``, ``Q4Block{scale, [u8; 16]}``, ``Q4_1Block{scale, min, [u8; 16]}`` and the
    ``QuantizedBlock`` enum over them).  The block is its packed bytes plus the type; ``scale`` /
    ``min`` read the fp16 header fields and ``dequantize`` expands the values."""
    quant_type: QuantType
    data: bytes
    layout: str = "ggml"

    def __post_init__(self):
        if len(self.data) != self.quant_type.bytes_per_block():
            raise QuantError(f"a {self.quant_type.value} block is {self.quant_type.bytes_per_block()} bytes, got {len(self.data)}")

    @classmethod
    def from_bytes(cls, quant_type: QuantType, data: bytes, layout: str = "ggml"):
        return cls(quant_type, bytes(data), layout)

    def to_bytes(self) -> bytes:
        return self.data

    def _half(self, offset: int) -> float:
        import struct
        return struct.unpack_from("<e", self.data, offset)[0]

    @property
    def scale(self) -> float | None:
        """fp16 scale ``d`` of the block (None for the unquantised types)."""
        return self._half(0) if self.quant_type.is_block_quantized() else None

    @property
    def min(self) -> float | None:
        """fp16 minimum ``m`` of the asymmetric types (Q4_1, Q5_1) and ``dmin`` of Q4_K."""
        return self._half(2) if self.quant_type in (QuantType.Q4_1, QuantType.Q5_1, QuantType.Q4_K) else None

    def dequantize(self) -> list:
        from .quantize import dequantize_tensor
        q = QuantizedTensor([self.quant_type.block_size()], self.quant_type, torch.frombuffer(bytearray(self.data), dtype=torch.uint8),
                            self.layout)
        return dequantize_tensor(q).tolist()


DEFAULT_BLOCK_SIZE = 32        # values per block of the Q8_0 / Q4_x / Q5_x types
MAX_BLOCK_SIZE = 256           # values per Q4_K super-block


def _f16_bytes(x: float) -> bytes:
    import struct
    return struct.pack("<e", float(x))


def _f16_round(x: float) -> float:
    import struct
    return struct.unpack("<e", struct.pack("<e", float(x)))[0]


@dataclasses.dataclass
class Q8Block:
    """fp16 scale + 32 signed bytes (types.rs:125-160); value i = scale * data[i]."""
    scale: float
    data: list

    def __post_init__(self):
        self.scale, self.data = _f16_round(self.scale), [int(v) for v in self.data]
        if len(self.data) != 32 or any(not -128 <= v <= 127 for v in self.data):
            raise QuantError("a Q8 block holds 32 values in -128..127")

    @classmethod
    def new(cls, scale, data): return cls(scale, data)
    def to_bytes(self) -> bytes: return _f16_bytes(self.scale) + bytes(v & 0xFF for v in self.data)

    @classmethod
    def from_bytes(cls, b: bytes):
        if len(b) < 34:
            return None
        import struct
        return cls(struct.unpack_from("<e", b, 0)[0], list(struct.unpack_from("<32b", b, 2)))

    def dequantize(self) -> list: return [self.scale * v for v in self.data]
    def as_block(self) -> QuantizedBlock: return QuantizedBlock(QuantType.Q8_0, self.to_bytes())


@dataclasses.dataclass
class Q4Block:
    """fp16 scale + 16 bytes of nibbles in the reference's adjacent-pair order (types.rs:162-215):
    byte i carries value 2i in its low and 2i+1 in its high nibble, each stored as value + 8."""
    scale: float
    data: bytes

    def __post_init__(self):
        self.scale, self.data = _f16_round(self.scale), bytes(self.data)
        if len(self.data) != 16:
            raise QuantError("a Q4 block holds 16 packed bytes")

    @classmethod
    def new(cls, scale, data): return cls(scale, data)

    def unpack(self) -> list:
        out = []
        for byte in self.data:
            out += [(byte & 0x0F) - 8, (byte >> 4) - 8]
        return out

    @staticmethod
    def pack(values) -> bytes:
        values = [int(v) for v in values]
        if len(values) != 32 or any(not -8 <= v <= 7 for v in values):
            raise QuantError("Q4 packs 32 values in -8..7")
        return bytes(((values[2 * i] + 8) & 0x0F) | (((values[2 * i + 1] + 8) & 0x0F) << 4) for i in range(16))

    def to_bytes(self) -> bytes: return _f16_bytes(self.scale) + self.data

    @classmethod
    def from_bytes(cls, b: bytes):
        if len(b) < 18:
            return None
        import struct
        return cls(struct.unpack_from("<e", b, 0)[0], bytes(b[2:18]))

    def dequantize(self) -> list: return [self.scale * v for v in self.unpack()]
    def as_block(self) -> QuantizedBlock: return QuantizedBlock(QuantType.Q4_0, self.to_bytes(), "adjacent")


@dataclasses.dataclass
class Q4_1Block:
    """fp16 scale, fp16 minimum and 16 bytes of unsigned nibbles in adjacent-pair order
    (types.rs:217-250); value i = min + scale * nibble i."""
    scale: float
    min: float
    data: bytes

    def __post_init__(self):
        self.scale, self.min, self.data = _f16_round(self.scale), _f16_round(self.min), bytes(self.data)
        if len(self.data) != 16:
            raise QuantError("a Q4_1 block holds 16 packed bytes")

    @classmethod
    def new(cls, scale, min, data): return cls(scale, min, data)

    def unpack(self) -> list:
        out = []
        for byte in self.data:
            out += [byte & 0x0F, byte >> 4]
        return out

    def to_bytes(self) -> bytes: return _f16_bytes(self.scale) + _f16_bytes(self.min) + self.data

    @classmethod
    def from_bytes(cls, b: bytes):
        if len(b) < 20:
            return None
        import struct
        return cls(struct.unpack_from("<e", b, 0)[0], struct.unpack_from("<e", b, 2)[0], bytes(b[4:20]))

    def dequantize(self) -> list: return [self.min + self.scale * v for v in self.unpack()]
    def as_block(self) -> QuantizedBlock: return QuantizedBlock(QuantType.Q4_1, self.to_bytes(), "adjacent")
