"""Readers and writers of the checkpoint containers.

* ``.axonml`` / ``.bin``: bincode 1.x of ``StateDict`` (crates/axonml-serialize/src/lib.rs:147-199),
  encoded/decoded by the C++ codec (``csrc/host/bincode.cpp``); byte-compatible with files the
  reference writes (HashMap order is arbitrary; f32 payloads).
* ``.json``: ``{"entries": {name: {"data": {"shape": [...], "values": [...]}, "requires_grad": b,
  "metadata": {...}}}, "metadata": {...}}`` (serde_json of the same structs).
* ``.safetensors``: the standard container (F32 / F16 / BF16 read, F32 or BF16 written); files from
  the reference's own writer, which stores shapes as ``"<name>.shape"`` metadata strings
  (lib.rs:244-303), are accepted too.
"""
from __future__ import annotations

import ctypes
import json
import struct

import numpy as np
import torch

from .. import _native as N
from .state_dict import StateDict, StateDictEntry, TensorData

_u64 = ctypes.c_uint64


def _lib():
    lib = N.host()
    if not getattr(lib, "_bc_typed", False):
        lib.ax_bc_writer_new.restype = ctypes.c_void_p
        lib.ax_bc_writer_data.restype = ctypes.c_void_p
        lib.ax_bc_writer_size.restype = ctypes.c_uint64
        lib.ax_bc_open_state_dict.restype = ctypes.c_void_p
        for f in ("ax_bc_count", "ax_bc_end", "ax_bc_meta_count", "ax_bc_meta_offset"):
            getattr(lib, f).restype = ctypes.c_uint64
        lib._bc_typed = True
    return lib


# ------------------------------------------------------------------ bincode: StateDict
def _write_map(lib, w, m: dict) -> None:
    lib.ax_bc_write_u64(ctypes.c_void_p(w), _u64(len(m)))
    for k, v in m.items():
        kb, vb = str(k).encode(), str(v).encode()
        lib.ax_bc_write_str(ctypes.c_void_p(w), kb, _u64(len(kb)))
        lib.ax_bc_write_str(ctypes.c_void_p(w), vb, _u64(len(vb)))


def _write_state_dict(lib, w, sd: StateDict) -> None:
    lib.ax_bc_write_u64(ctypes.c_void_p(w), _u64(len(sd)))
    for name, e in sd.entries():
        kb = name.encode()
        lib.ax_bc_write_str(ctypes.c_void_p(w), kb, _u64(len(kb)))
        vals = e.data.values.contiguous()
        shape = (ctypes.c_uint64 * len(e.data.shape))(*e.data.shape)
        lib.ax_bc_write_entry(ctypes.c_void_p(w), shape, _u64(len(e.data.shape)),
                              ctypes.c_void_p(vals.data_ptr()), _u64(vals.numel()),
                              ctypes.c_uint8(1 if e.requires_grad else 0))
        _write_map(lib, w, e.metadata)
    _write_map(lib, w, sd.metadata)


def _writer_bytes(lib, w) -> bytes:
    n = lib.ax_bc_writer_size(ctypes.c_void_p(w))
    return ctypes.string_at(lib.ax_bc_writer_data(ctypes.c_void_p(w)), n)


def encode_state_dict(sd: StateDict) -> bytes:
    lib = _lib()
    w = lib.ax_bc_writer_new()
    try:
        _write_state_dict(lib, w, sd)
        return _writer_bytes(lib, w)
    finally:
        lib.ax_bc_writer_free(ctypes.c_void_p(w))


def _read_str(buf: memoryview, pos: int):
    n = struct.unpack_from("<Q", buf, pos)[0]
    return bytes(buf[pos + 8:pos + 8 + n]).decode(), pos + 8 + n


def _read_map(buf: memoryview, pos: int, n: int):
    out = {}
    for _ in range(n):
        k, pos = _read_str(buf, pos)
        v, pos = _read_str(buf, pos)
        out[k] = v
    return out, pos


def decode_state_dict(data: bytes, start: int = 0):
    """Returns ``(StateDict, end_offset)``."""
    from ..core.error import SerializationError
    lib = _lib()
    raw = np.frombuffer(data, dtype=np.uint8)
    h = lib.ax_bc_open_state_dict(ctypes.c_void_p(raw.ctypes.data), _u64(len(data)), _u64(start))
    if not h:
        raise SerializationError("not a bincode StateDict (truncated or corrupt)")
    try:
        buf = memoryview(data)
        sd = StateDict()
        out = (ctypes.c_uint64 * 9)()
        for i in range(lib.ax_bc_count(ctypes.c_void_p(h))):
            lib.ax_bc_entry(ctypes.c_void_p(h), _u64(i), out)
            key_off, key_len, ndim, shape_off, nvals, data_off, rg, nmeta, meta_off = list(out)
            name = bytes(buf[key_off:key_off + key_len]).decode()
            shape = list(struct.unpack_from(f"<{ndim}Q", buf, shape_off)) if ndim else []
            vals = torch.from_numpy(np.frombuffer(data, dtype="<f4", count=nvals, offset=data_off).copy())
            meta, _ = _read_map(buf, meta_off, nmeta)
            sd.insert_entry(name, StateDictEntry(TensorData(shape, vals), bool(rg), meta))
        sd.metadata, _ = _read_map(buf, lib.ax_bc_meta_offset(ctypes.c_void_p(h)),
                                   lib.ax_bc_meta_count(ctypes.c_void_p(h)))
        return sd, int(lib.ax_bc_end(ctypes.c_void_p(h)))
    finally:
        lib.ax_bc_close(ctypes.c_void_p(h))


# ------------------------------------------------------------------ JSON
def state_dict_to_json(sd: StateDict) -> str:
    obj = {"entries": {k: {"data": {"shape": e.data.shape, "values": e.data.values.tolist()},
                           "requires_grad": e.requires_grad, "metadata": e.metadata}
                       for k, e in sd.entries()}, "metadata": sd.metadata}
    return json.dumps(obj, indent=2)


def state_dict_from_json(text: str) -> StateDict:
    obj = json.loads(text)
    sd = StateDict()
    for k, e in obj.get("entries", {}).items():
        sd.insert_entry(k, StateDictEntry(TensorData(list(e["data"]["shape"]),
                                                     torch.tensor(e["data"]["values"], dtype=torch.float32)),
                                          bool(e.get("requires_grad", True)), dict(e.get("metadata", {}))))
    sd.metadata = dict(obj.get("metadata", {}))
    return sd


# ------------------------------------------------------------------ safetensors
_ST_DTYPES = {"F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
              "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
              "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "BOOL": (torch.bool, 1)}
_ST_NAMES = {v[0]: k for k, v in _ST_DTYPES.items()}


def safetensors_dumps(tensors: dict, metadata: dict | None = None) -> bytes:
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    return struct.pack("<Q", len(hj)) + hj + b"".join(blobs)


def safetensors_loads(data: bytes):
    """Returns ``(tensors, metadata)``; tensors keep their stored dtype."""
    from ..core.error import SerializationError
    if len(data) < 8:
        raise SerializationError("safetensors file too short")
    n = struct.unpack_from("<Q", data, 0)[0]
    if n > len(data) - 8:
        raise SerializationError("safetensors header length exceeds the file")
    header = json.loads(data[8:8 + n].decode())
    meta = header.pop("__metadata__", {}) or {}
    base = 8 + n
    out = {}
    for name, info in header.items():
        dt, sz = _ST_DTYPES[info["dtype"]]
        a, b = info["data_offsets"]
        shape = info.get("shape")
        if shape is None or (shape == [] and f"{name}.shape" in meta):
            shape = json.loads(meta[f"{name}.shape"])       # the reference's own writer
        buf = bytearray(data[base + a:base + b])
        t = torch.frombuffer(buf, dtype=dt) if buf else torch.empty(0, dtype=dt)
        out[name] = t.view(shape)
    return out, meta
