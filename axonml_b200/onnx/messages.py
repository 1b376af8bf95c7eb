"""ONNX protobuf messages as objects.

Parity: crates/axonml-onnx/src/proto.rs (``TensorDataType`` with ``size_bytes`` / ``from_i32``,
``Dimension`` fixed or symbolic, ``TensorShape``, ``TensorType``, ``TypeProto``, ``ValueInfo``,
``TensorProto`` with typed accessors, ``AttributeType``, ``AttributeProto`` with the ``int`` /
``float`` / ``ints`` constructors, ``NodeProto`` with attribute lookups, ``GraphProto`` with
``get_initializer`` / ``initializer_map``, ``OperatorSetIdProto``, ``StringStringEntry``,
``ModelProto`` with ``opset_version``).  Every message reads itself from protobuf bytes
(``from_bytes``) and writes itself back (``to_bytes``) with the field numbers of onnx.proto3, so a
file can be inspected, edited and saved without the ``onnx`` package."""
from __future__ import annotations

import dataclasses
import enum
import struct

import numpy as np
import torch

from . import proto as P

ONNX_IR_VERSION = 8
SUPPORTED_OPSET_VERSION = 17


class TensorDataType(enum.IntEnum):
    Undefined = 0
    Float = 1
    Uint8 = 2
    Int8 = 3
    Uint16 = 4
    Int16 = 5
    Int32 = 6
    Int64 = 7
    String = 8
    Bool = 9
    Float16 = 10
    Double = 11
    Uint32 = 12
    Uint64 = 13
    Complex64 = 14
    Complex128 = 15
    Bfloat16 = 16

    def size_bytes(self) -> int:
        return _SIZES.get(self, 0)

    @classmethod
    def from_i32(cls, value: int):
        try:
            return cls(value)
        except ValueError:
            return None

    def numpy_dtype(self):
        return _NUMPY.get(self)

    def torch_dtype(self):
        return _TORCH.get(self)


_T = TensorDataType
_SIZES = {_T.Float: 4, _T.Uint8: 1, _T.Int8: 1, _T.Uint16: 2, _T.Int16: 2, _T.Int32: 4, _T.Int64: 8, _T.Bool: 1, _T.Float16: 2,
          _T.Double: 8, _T.Uint32: 4, _T.Uint64: 8, _T.Complex64: 8, _T.Complex128: 16, _T.Bfloat16: 2}
_NUMPY = {_T.Float: "<f4", _T.Uint8: "u1", _T.Int8: "i1", _T.Uint16: "<u2", _T.Int16: "<i2", _T.Int32: "<i4", _T.Int64: "<i8",
          _T.Bool: "?", _T.Float16: "<f2", _T.Double: "<f8", _T.Uint32: "<u4", _T.Uint64: "<u8"}
_TORCH = {_T.Float: torch.float32, _T.Uint8: torch.uint8, _T.Int8: torch.int8, _T.Int16: torch.int16, _T.Int32: torch.int32,
          _T.Int64: torch.int64, _T.Bool: torch.bool, _T.Float16: torch.float16, _T.Double: torch.float64, _T.Bfloat16: torch.bfloat16}


class AttributeType(enum.IntEnum):
    Undefined = 0
    Float = 1
    Int = 2
    String = 3
    Tensor = 4
    Graph = 5
    Floats = 6
    Ints = 7
    Strings = 8
    Tensors = 9
    Graphs = 10
    SparseTensor = 11
    SparseTensors = 12


def _s(v: bytes) -> str:
    return v.decode("utf-8", errors="replace")


def _floats(wt, v) -> list:
    return list(struct.unpack(f"<{len(v) // 4}f", v)) if wt == 2 else [struct.unpack("<f", v)[0]]


def _doubles(wt, v) -> list:
    return list(struct.unpack(f"<{len(v) // 8}d", v)) if wt == 2 else [struct.unpack("<d", v)[0]]


def _ints(wt, v) -> list:
    return P.packed_ints(v) if wt == 2 else [P.signed(v)]


def _opt_str(field: int, s) -> bytes:
    return P.enc_str(field, s) if s is not None else b""


@dataclasses.dataclass
class Dimension:
    dim_value: int | None = None
    dim_param: str | None = None

    @classmethod
    def fixed(cls, value: int): return cls(int(value), None)
    @classmethod
    def dynamic(cls, name: str): return cls(None, name)
    def value(self): return self.dim_value

    @classmethod
    def from_bytes(cls, buf: bytes):
        d = cls()
        for f, _, v in P.parse(buf):
            if f == 1: d.dim_value = P.signed(v)
            elif f == 2: d.dim_param = _s(v)
        return d

    def to_bytes(self) -> bytes:
        return P.enc_varint(1, self.dim_value) if self.dim_value is not None else _opt_str(2, self.dim_param)


@dataclasses.dataclass
class TensorShape:
    dims: list = dataclasses.field(default_factory=list)

    @classmethod
    def from_dims(cls, dims):
        """Negative extents become dynamic dimensions."""
        return cls([Dimension.fixed(d) if int(d) >= 0 else Dimension.dynamic(f"dim_{i}") for i, d in enumerate(dims)])

    def to_vec(self) -> list: return [d.dim_value for d in self.dims]

    @classmethod
    def from_bytes(cls, buf: bytes):
        return cls([Dimension.from_bytes(v) for f, _, v in P.parse(buf) if f == 1])

    def to_bytes(self) -> bytes:
        return b"".join(P.enc_bytes(1, d.to_bytes()) for d in self.dims)


@dataclasses.dataclass
class TensorType:
    elem_type: int = int(TensorDataType.Float)
    shape: TensorShape | None = None

    @classmethod
    def from_bytes(cls, buf: bytes):
        t = cls(0, None)
        for f, _, v in P.parse(buf):
            if f == 1: t.elem_type = v
            elif f == 2: t.shape = TensorShape.from_bytes(v)
        return t

    def to_bytes(self) -> bytes:
        return P.enc_varint(1, int(self.elem_type)) + (P.enc_bytes(2, self.shape.to_bytes()) if self.shape is not None else b"")


@dataclasses.dataclass
class TypeProto:
    tensor_type: TensorType | None = None

    @classmethod
    def from_bytes(cls, buf: bytes):
        return cls(next((TensorType.from_bytes(v) for f, _, v in P.parse(buf) if f == 1), None))

    def to_bytes(self) -> bytes:
        return P.enc_bytes(1, self.tensor_type.to_bytes()) if self.tensor_type is not None else b""


@dataclasses.dataclass
class ValueInfo:
    name: str = ""
    type: TypeProto | None = None
    doc_string: str | None = None

    @classmethod
    def tensor(cls, name: str, shape, elem_type: int = int(TensorDataType.Float)):
        dims = [Dimension.dynamic(d) if isinstance(d, str) else Dimension.fixed(d) for d in shape]
        return cls(name, TypeProto(TensorType(int(elem_type), TensorShape(dims))))

    def shape(self):
        """List of extents (None where symbolic), or None when the value has no tensor type."""
        tt = self.type.tensor_type if self.type else None
        return tt.shape.to_vec() if tt and tt.shape else None

    @classmethod
    def from_bytes(cls, buf: bytes):
        vi = cls()
        for f, _, v in P.parse(buf):
            if f == 1: vi.name = _s(v)
            elif f == 2: vi.type = TypeProto.from_bytes(v)
            elif f == 3: vi.doc_string = _s(v)
        return vi

    def to_bytes(self) -> bytes:
        return P.enc_str(1, self.name) + (P.enc_bytes(2, self.type.to_bytes()) if self.type else b"") + _opt_str(3, self.doc_string)


@dataclasses.dataclass
class TensorProto:
    name: str = ""
    dims: list = dataclasses.field(default_factory=list)
    data_type: int = int(TensorDataType.Float)
    raw_data: bytes = b""
    float_data: list = dataclasses.field(default_factory=list)
    int32_data: list = dataclasses.field(default_factory=list)
    int64_data: list = dataclasses.field(default_factory=list)
    double_data: list = dataclasses.field(default_factory=list)
    doc_string: str | None = None

    @classmethod
    def float(cls, name: str, dims, data):
        return cls(name, [int(d) for d in dims], int(TensorDataType.Float), float_data=[float(x) for x in data])

    @classmethod
    def from_tensor(cls, name: str, t: torch.Tensor):
        """Tensor stored as little-endian ``raw_data``."""
        kinds = {v: k for k, v in _TORCH.items()}
        dt = kinds.get(t.dtype)
        if dt is None or dt is TensorDataType.Bfloat16:
            t, dt = t.float(), TensorDataType.Float
        arr = t.detach().cpu().contiguous().numpy()
        return cls(name, list(arr.shape), int(dt), raw_data=arr.astype(arr.dtype.newbyteorder("<")).tobytes())

    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def to_numpy(self) -> np.ndarray:
        dt = TensorDataType.from_i32(self.data_type)
        np_dt = dt.numpy_dtype() if dt is not None else None
        if np_dt is None:
            raise ValueError(f"tensor {self.name!r}: data type {self.data_type} has no array form")
        if self.raw_data:
            arr = np.frombuffer(self.raw_data, dtype=np_dt).copy()
        elif self.float_data:
            arr = np.asarray(self.float_data, dtype=np.float32)
        elif self.double_data:
            arr = np.asarray(self.double_data, dtype=np.float64)
        elif self.int64_data:
            arr = np.asarray(self.int64_data, dtype=np.int64)
        elif self.int32_data:       # also carries the narrow integer types, bool and fp16 bit patterns
            arr = np.asarray(self.int32_data, dtype=np.int32)
            arr = arr.astype(np.uint16).view(np.float16) if dt is TensorDataType.Float16 else arr.astype(np_dt)
        else:
            arr = np.zeros(0, dtype=np_dt)
        return arr.astype(np_dt, copy=False).reshape(self.dims)

    def to_tensor(self) -> torch.Tensor:
        return torch.from_numpy(self.to_numpy())

    def get_float_data(self) -> list:
        return self.to_numpy().astype(np.float32).reshape(-1).tolist()

    def get_int64_data(self) -> list:
        return self.to_numpy().astype(np.int64).reshape(-1).tolist()

    @classmethod
    def from_bytes(cls, buf: bytes):
        t = cls()
        for f, wt, v in P.parse(buf):
            if f == 1: t.dims += _ints(wt, v)
            elif f == 2: t.data_type = v
            elif f == 4: t.float_data += _floats(wt, v)
            elif f == 5: t.int32_data += _ints(wt, v)
            elif f == 7: t.int64_data += _ints(wt, v)
            elif f == 8: t.name = _s(v)
            elif f == 9: t.raw_data = bytes(v)
            elif f == 10: t.double_data += _doubles(wt, v)
            elif f == 12: t.doc_string = _s(v)
        return t

    def to_bytes(self) -> bytes:
        b = b"".join(P.enc_varint(1, int(d)) for d in self.dims) + P.enc_varint(2, int(self.data_type))
        if self.float_data:
            b += P.enc_bytes(4, struct.pack(f"<{len(self.float_data)}f", *self.float_data))
        if self.int32_data:
            b += P.enc_bytes(5, b"".join(P._varint(int(x)) for x in self.int32_data))
        if self.int64_data:
            b += P.enc_bytes(7, b"".join(P._varint(int(x)) for x in self.int64_data))
        b += P.enc_str(8, self.name)
        if self.raw_data:
            b += P.enc_bytes(9, self.raw_data)
        if self.double_data:
            b += P.enc_bytes(10, struct.pack(f"<{len(self.double_data)}d", *self.double_data))
        return b + _opt_str(12, self.doc_string)


@dataclasses.dataclass
class AttributeProto:
    name: str = ""
    type: int = int(AttributeType.Undefined)
    f: float | None = None
    i: int | None = None
    s: bytes | None = None
    t: TensorProto | None = None
    floats: list = dataclasses.field(default_factory=list)
    ints: list = dataclasses.field(default_factory=list)
    strings: list = dataclasses.field(default_factory=list)
    doc_string: str | None = None

    @classmethod
    def int(cls, name: str, value: int): return cls(name, AttributeType.Int.value, i=value)
    @classmethod
    def float(cls, name: str, value: float): return cls(name, AttributeType.Float.value, f=value)
    @classmethod
    def string(cls, name: str, value: str): return cls(name, AttributeType.String.value, s=value.encode())
    @classmethod
    def ints_(cls, name: str, values): return cls(name, AttributeType.Ints.value, ints=[v for v in values])
    @classmethod
    def floats_(cls, name: str, values): return cls(name, AttributeType.Floats.value, floats=[v for v in values])
    @classmethod
    def tensor(cls, name: str, value: TensorProto): return cls(name, AttributeType.Tensor.value, t=value)

    def get_string(self):
        return _s(self.s) if self.s is not None else None

    def value(self):
        """The attribute as a plain Python value (tensor attributes as torch tensors)."""
        kind = AttributeType(self.type) if self.type in AttributeType._value2member_map_ else AttributeType.Undefined
        if kind is AttributeType.Float or (kind is AttributeType.Undefined and self.f is not None): return self.f
        if kind is AttributeType.Int or (kind is AttributeType.Undefined and self.i is not None): return self.i
        if kind is AttributeType.String or (kind is AttributeType.Undefined and self.s is not None): return self.get_string()
        if kind is AttributeType.Tensor or (kind is AttributeType.Undefined and self.t is not None): return self.t.to_tensor()
        if kind is AttributeType.Floats or (kind is AttributeType.Undefined and self.floats): return list(self.floats)
        if kind is AttributeType.Ints or (kind is AttributeType.Undefined and self.ints): return list(self.ints)
        if kind is AttributeType.Strings or (kind is AttributeType.Undefined and self.strings): return [_s(x) for x in self.strings]
        return None

    @classmethod
    def from_bytes(cls, buf: bytes):
        a = cls()
        for f, wt, v in P.parse(buf):
            if f == 1: a.name = _s(v)
            elif f == 2: a.f = struct.unpack("<f", v)[0]
            elif f == 3: a.i = P.signed(v)
            elif f == 4: a.s = bytes(v)
            elif f == 5: a.t = TensorProto.from_bytes(v)
            elif f == 7: a.floats += _floats(wt, v)
            elif f == 8: a.ints += _ints(wt, v)
            elif f == 9: a.strings.append(bytes(v))
            elif f == 13: a.doc_string = _s(v)
            elif f == 20: a.type = v
        return a

    def to_bytes(self) -> bytes:
        b = P.enc_str(1, self.name)
        if self.f is not None: b += P.enc_float(2, self.f)
        if self.i is not None: b += P.enc_varint(3, self.i)
        if self.s is not None: b += P.enc_bytes(4, self.s)
        if self.t is not None: b += P.enc_bytes(5, self.t.to_bytes())
        b += b"".join(P.enc_float(7, x) for x in self.floats) + b"".join(P.enc_varint(8, x) for x in self.ints)
        b += b"".join(P.enc_bytes(9, x) for x in self.strings) + _opt_str(13, self.doc_string)
        return b + P.enc_varint(20, int(self.type))


# the reference's constructor names; ``ints`` / ``floats`` are also field names of the dataclass,
# so the class-level constructors carry a trailing underscore and these aliases keep the spelling
AttributeProto.make_ints = AttributeProto.ints_
AttributeProto.make_floats = AttributeProto.floats_


@dataclasses.dataclass
class NodeProto:
    input: list = dataclasses.field(default_factory=list)
    output: list = dataclasses.field(default_factory=list)
    name: str | None = None
    op_type: str = ""
    domain: str | None = None
    attribute: list = dataclasses.field(default_factory=list)
    doc_string: str | None = None

    def get_attribute(self, name: str):
        return next((a for a in self.attribute if a.name == name), None)

    def get_int(self, name: str, default=None):
        a = self.get_attribute(name)
        return a.i if a is not None and a.i is not None else default

    def get_float(self, name: str, default=None):
        a = self.get_attribute(name)
        return a.f if a is not None and a.f is not None else default

    def get_ints(self, name: str, default=None):
        a = self.get_attribute(name)
        return list(a.ints) if a is not None and (a.ints or a.type == AttributeType.Ints) else default

    def get_string(self, name: str, default=None):
        a = self.get_attribute(name)
        return a.get_string() if a is not None and a.s is not None else default

    def attrs(self) -> dict:
        return {a.name: a.value() for a in self.attribute}

    @classmethod
    def from_bytes(cls, buf: bytes):
        n = cls()
        for f, _, v in P.parse(buf):
            if f == 1: n.input.append(_s(v))
            elif f == 2: n.output.append(_s(v))
            elif f == 3: n.name = _s(v)
            elif f == 4: n.op_type = _s(v)
            elif f == 5: n.attribute.append(AttributeProto.from_bytes(v))
            elif f == 6: n.doc_string = _s(v)
            elif f == 7: n.domain = _s(v)
        return n

    def to_bytes(self) -> bytes:
        b = b"".join(P.enc_str(1, x) for x in self.input) + b"".join(P.enc_str(2, x) for x in self.output)
        b += _opt_str(3, self.name) + P.enc_str(4, self.op_type) + b"".join(P.enc_bytes(5, a.to_bytes()) for a in self.attribute)
        return b + _opt_str(6, self.doc_string) + _opt_str(7, self.domain)


@dataclasses.dataclass
class GraphProto:
    node: list = dataclasses.field(default_factory=list)
    name: str | None = None
    initializer: list = dataclasses.field(default_factory=list)
    sparse_initializer: list = dataclasses.field(default_factory=list)
    input: list = dataclasses.field(default_factory=list)
    output: list = dataclasses.field(default_factory=list)
    value_info: list = dataclasses.field(default_factory=list)
    doc_string: str | None = None

    def get_initializer(self, name: str):
        return next((t for t in self.initializer if t.name == name), None)

    def initializer_map(self) -> dict:
        return {t.name: t for t in self.initializer}

    def graph_inputs(self) -> list:
        """Inputs that are not initializers (what a caller has to feed)."""
        have = {t.name for t in self.initializer}
        return [v for v in self.input if v.name not in have]

    @classmethod
    def from_bytes(cls, buf: bytes):
        g = cls()
        for f, _, v in P.parse(buf):
            if f == 1: g.node.append(NodeProto.from_bytes(v))
            elif f == 2: g.name = _s(v)
            elif f == 5: g.initializer.append(TensorProto.from_bytes(v))
            elif f == 10: g.doc_string = _s(v)
            elif f == 11: g.input.append(ValueInfo.from_bytes(v))
            elif f == 12: g.output.append(ValueInfo.from_bytes(v))
            elif f == 13: g.value_info.append(ValueInfo.from_bytes(v))
        return g

    def to_bytes(self) -> bytes:
        b = b"".join(P.enc_bytes(1, n.to_bytes()) for n in self.node) + _opt_str(2, self.name)
        b += b"".join(P.enc_bytes(5, t.to_bytes()) for t in self.initializer) + _opt_str(10, self.doc_string)
        b += b"".join(P.enc_bytes(11, v.to_bytes()) for v in self.input) + b"".join(P.enc_bytes(12, v.to_bytes()) for v in self.output)
        return b + b"".join(P.enc_bytes(13, v.to_bytes()) for v in self.value_info)


@dataclasses.dataclass
class OperatorSetIdProto:
    domain: str | None = None
    version: int = SUPPORTED_OPSET_VERSION

    @classmethod
    def from_bytes(cls, buf: bytes):
        o = cls(None, 0)
        for f, _, v in P.parse(buf):
            if f == 1: o.domain = _s(v)
            elif f == 2: o.version = P.signed(v)
        return o

    def to_bytes(self) -> bytes:
        return _opt_str(1, self.domain) + P.enc_varint(2, self.version)


@dataclasses.dataclass
class StringStringEntry:
    key: str = ""
    value: str = ""

    @classmethod
    def from_bytes(cls, buf: bytes):
        e = cls()
        for f, _, v in P.parse(buf):
            if f == 1: e.key = _s(v)
            elif f == 2: e.value = _s(v)
        return e

    def to_bytes(self) -> bytes:
        return P.enc_str(1, self.key) + P.enc_str(2, self.value)


@dataclasses.dataclass
class ModelProto:
    ir_version: int = ONNX_IR_VERSION
    opset_import: list = dataclasses.field(default_factory=list)
    producer_name: str | None = None
    producer_version: str | None = None
    domain: str | None = None
    model_version: int | None = None
    doc_string: str | None = None
    graph: GraphProto | None = None
    metadata_props: list = dataclasses.field(default_factory=list)

    def opset_version(self) -> int:
        """Version of the default (empty or ``ai.onnx``) domain; the supported version when none is listed."""
        for o in self.opset_import:
            if not o.domain or o.domain == "ai.onnx":
                return o.version
        return SUPPORTED_OPSET_VERSION

    def metadata(self) -> dict:
        return {e.key: e.value for e in self.metadata_props}

    @classmethod
    def from_bytes(cls, buf: bytes):
        m = cls(ir_version=0)
        for f, _, v in P.parse(buf):
            if f == 1: m.ir_version = P.signed(v)
            elif f == 2: m.producer_name = _s(v)
            elif f == 3: m.producer_version = _s(v)
            elif f == 4: m.domain = _s(v)
            elif f == 5: m.model_version = P.signed(v)
            elif f == 6: m.doc_string = _s(v)
            elif f == 7: m.graph = GraphProto.from_bytes(v)
            elif f == 8: m.opset_import.append(OperatorSetIdProto.from_bytes(v))
            elif f == 14: m.metadata_props.append(StringStringEntry.from_bytes(v))
        return m

    @classmethod
    def load(cls, path):
        with open(path, "rb") as f:
            return cls.from_bytes(f.read())

    def to_bytes(self) -> bytes:
        b = P.enc_varint(1, self.ir_version) + _opt_str(2, self.producer_name) + _opt_str(3, self.producer_version) + _opt_str(4, self.domain)
        if self.model_version is not None:
            b += P.enc_varint(5, self.model_version)
        b += _opt_str(6, self.doc_string) + (P.enc_bytes(7, self.graph.to_bytes()) if self.graph is not None else b"")
        b += b"".join(P.enc_bytes(8, o.to_bytes()) for o in self.opset_import)
        return b + b"".join(P.enc_bytes(14, e.to_bytes()) for e in self.metadata_props)

    def save(self, path) -> None:
        with open(path, "wb") as f:
            f.write(self.to_bytes())
