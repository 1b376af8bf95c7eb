"""GGUF v3 container reader and writer (public GGUF specification): header, typed key/value
metadata, tensor directory (dimensions stored innermost-first), 32-byte aligned tensor data in
GGML block layouts (F32, F16, BF16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K).  The reader memory-maps
the file, so opening an 8B-parameter model costs no copy until a tensor is requested."""
from __future__ import annotations

import mmap
import struct

import numpy as np
import torch

from .quantize import dequantize_tensor, quantize_tensor
from .types import QuantError, QuantizedTensor, QuantType

MAGIC = b"GGUF"
ALIGN = 32
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


def _vtype(v):
    if isinstance(v, bool): return 7
    if isinstance(v, int): return 4 if 0 <= v < 2 ** 32 else (11 if v < 0 else 10)
    if isinstance(v, float): return 6
    if isinstance(v, str): return 8
    if isinstance(v, (list, tuple)): return 9
    raise QuantError(f"unsupported GGUF metadata value {v!r}")


def _wstr(out: bytearray, s: str) -> None:
    b = s.encode()
    out += struct.pack("<Q", len(b)) + b


def _wval(out: bytearray, v, t=None) -> None:
    t = _vtype(v) if t is None else t
    if t == 8:
        _wstr(out, v)
    elif t == 9:
        et = _vtype(v[0]) if len(v) else 4
        out += struct.pack("<IQ", et, len(v))
        for x in v:
            _wval(out, x, et)
    else:
        out += struct.pack(_SCALAR[t], v)


def write_gguf(path, tensors: dict, metadata: dict | None = None, quant: dict | None = None,
               default_quant: QuantType | None = None) -> None:
    """``tensors``: name -> torch.Tensor or QuantizedTensor.  ``quant``: per-name QuantType for plain
    tensors; ``default_quant`` applies to 2-D tensors whose row length fits the block size."""
    metadata = dict(metadata or {})
    metadata.setdefault("general.architecture", "llama")
    metadata.setdefault("general.alignment", ALIGN)
    entries = []
    for name, t in tensors.items():
        if isinstance(t, QuantizedTensor):
            q = t
        else:
            qt = (quant or {}).get(name)
            if qt is None:
                qt = default_quant if (default_quant is not None and t.dim() == 2
                                       and t.shape[-1] % default_quant.block_size() == 0) else QuantType.F32
            q = quantize_tensor(t, qt)
        entries.append((name, q))
    head = bytearray(MAGIC + struct.pack("<IQQ", 3, len(entries), len(metadata)))
    for k, v in metadata.items():
        _wstr(head, k)
        t = _vtype(v)
        head += struct.pack("<I", t)
        _wval(head, v, t)
    off, infos = 0, bytearray()
    offsets = []
    for name, q in entries:
        _wstr(infos, name)
        dims = list(reversed(q.shape)) or [1]
        infos += struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims)
        infos += struct.pack("<IQ", q.quant_type.ggml_type(), off)
        offsets.append(off)
        off += (q.size_bytes() + ALIGN - 1) // ALIGN * ALIGN
    pre = len(head) + len(infos)
    pad = (ALIGN - pre % ALIGN) % ALIGN
    with open(path, "wb") as f:
        f.write(head)
        f.write(infos)
        f.write(b"\0" * pad)
        for (name, q), o in zip(entries, offsets):
            raw = q.data.detach().cpu().contiguous().numpy().tobytes()
            f.write(raw)
            f.write(b"\0" * ((ALIGN - len(raw) % ALIGN) % ALIGN))


class GGUFFile:
    def __init__(self, path):
        self.path = str(path)
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.metadata: dict = {}
        self.tensors: dict = {}
        self._parse()

    def close(self) -> None:
        try:
            self._mm.close()
        finally:
            self._f.close()

    def _parse(self) -> None:
        mm = self._mm
        if mm[:4] != MAGIC:
            raise QuantError("not a GGUF file")
        version, n_tensors, n_kv = struct.unpack_from("<IQQ", mm, 4)
        if version not in (2, 3):
            raise QuantError(f"unsupported GGUF version {version}")
        self.version = version
        pos = 24

        def rstr():
            nonlocal pos
            n = struct.unpack_from("<Q", mm, pos)[0]
            s = bytes(mm[pos + 8:pos + 8 + n]).decode("utf-8", "replace")
            pos += 8 + n
            return s

        def rval(t):
            nonlocal pos
            if t == 8:
                return rstr()
            if t == 9:
                et, n = struct.unpack_from("<IQ", mm, pos)
                pos += 12
                if et in _SCALAR and et != 7:
                    fmt = _SCALAR[et]
                    sz = struct.calcsize(fmt)
                    arr = np.frombuffer(mm, dtype=np.dtype(fmt[1]).newbyteorder("<"), count=n, offset=pos)
                    pos += n * sz
                    return arr.tolist()
                return [rval(et) for _ in range(n)]
            fmt = _SCALAR[t]
            v = struct.unpack_from(fmt, mm, pos)[0]
            pos += struct.calcsize(fmt)
            return v
        for _ in range(n_kv):
            k = rstr()
            t = struct.unpack_from("<I", mm, pos)[0]
            pos += 4
            self.metadata[k] = rval(t)
        infos = []
        for _ in range(n_tensors):
            name = rstr()
            nd = struct.unpack_from("<I", mm, pos)[0]
            pos += 4
            dims = struct.unpack_from(f"<{nd}Q", mm, pos)
            pos += 8 * nd
            typ, off = struct.unpack_from("<IQ", mm, pos)
            pos += 12
            infos.append((name, list(reversed(dims)), typ, off))
        align = int(self.metadata.get("general.alignment", ALIGN))
        self.data_start = (pos + align - 1) // align * align
        for name, shape, typ, off in infos:
            qt = QuantType.from_ggml_type(typ)
            n = 1
            for s in shape:
                n *= s
            nbytes = n // qt.block_size() * qt.bytes_per_block()
            self.tensors[name] = (shape, qt, self.data_start + off, nbytes)

    def tensor_names(self): return list(self.tensors)

    def tensor_info(self, name: str) -> dict:
        """``{"shape", "type" (storage type name), "numel", "nbytes"}`` of one tensor."""
        shape, qt, _, nbytes = self.tensors[name]
        n = 1
        for d in shape:
            n *= d
        return {"shape": list(shape), "type": qt.value, "numel": n, "nbytes": nbytes}

    def quantized(self, name: str, device=None) -> QuantizedTensor:
        shape, qt, off, nbytes = self.tensors[name]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")        # read-only mmap: the tensor is copied right below
            data = torch.frombuffer(self._mm, dtype=torch.uint8, count=nbytes, offset=off)
        data = data.to(device) if device is not None else data.clone()
        return QuantizedTensor(shape, qt, data)

    def tensor(self, name: str, dtype=torch.float32) -> torch.Tensor:
        return dequantize_tensor(self.quantized(name), dtype)


def read_gguf(path) -> GGUFFile:
    return GGUFFile(path)
