"""Minimal protobuf wire codec for the ONNX messages this package reads and writes
(hand-rolled like the reference's, crates/axonml-onnx/src/proto.rs; no ``onnx`` dependency)."""
from __future__ import annotations

import struct


def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def enc_varint(field: int, v: int) -> bytes: return _varint(field << 3) + _varint(v)
def enc_bytes(field: int, b: bytes) -> bytes: return _varint((field << 3) | 2) + _varint(len(b)) + b
def enc_str(field: int, s: str) -> bytes: return enc_bytes(field, s.encode())
def enc_float(field: int, f: float) -> bytes: return _varint((field << 3) | 5) + struct.pack("<f", f)


def parse(buf: bytes) -> list:
    """-> list of (field, wire_type, value); value = int | bytes."""
    out, i, n = [], 0, len(buf)
    while i < n:
        key, i = _read_varint(buf, i)
        field, wt = key >> 3, key & 7
        if wt == 0:
            v, i = _read_varint(buf, i)
        elif wt == 1:
            v, i = buf[i:i + 8], i + 8
        elif wt == 2:
            ln, i = _read_varint(buf, i)
            v, i = buf[i:i + ln], i + ln
        elif wt == 5:
            v, i = buf[i:i + 4], i + 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
        out.append((field, wt, v))
    return out


def _read_varint(buf, i):
    shift = v = 0
    while True:
        b = buf[i]
        i += 1
        v |= (b & 0x7F) << shift
        if not b & 0x80:
            return v, i
        shift += 7


def signed(v: int) -> int:
    return v - (1 << 64) if v >= 1 << 63 else v


def packed_ints(b: bytes) -> list:
    out, i = [], 0
    while i < len(b):
        v, i = _read_varint(b, i)
        out.append(signed(v))
    return out


# ONNX TensorProto.DataType
FLOAT, UINT8, INT8, INT32, INT64, BOOL, FLOAT16, DOUBLE, BFLOAT16 = 1, 2, 3, 6, 7, 9, 10, 11, 16
