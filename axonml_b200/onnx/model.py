"""ONNX import and execution (crates/axonml-onnx/src/parser.rs:35-53, model.rs:22-162,
operators.rs): ``import_onnx`` parses a ModelProto into an ``OnnxModel`` whose ``forward`` runs
the graph over torch tensors (on the GPU when the inputs are there).  Operators: Relu Sigmoid Tanh
Softmax LeakyRelu Gelu Add Sub Mul Div MatMul Gemm Sqrt Pow Exp Log Reshape Transpose Flatten
Squeeze Unsqueeze Concat Gather ReduceSum ReduceMean ReduceMax Conv MaxPool AveragePool
BatchNormalization Dropout Constant Identity Cast Shape Equal Greater Less Clip (the reference's 39)
plus GlobalAveragePool, Neg, Abs, Where, Erf, LayerNormalization."""
from __future__ import annotations

import dataclasses
import struct

import numpy as np
import torch
import torch.nn.functional as F

from . import proto as P

_NP = {P.FLOAT: "<f4", P.INT64: "<i8", P.INT32: "<i4", P.DOUBLE: "<f8", P.UINT8: "u1", P.INT8: "i1", P.BOOL: "?", P.FLOAT16: "<f2"}
_TORCH = {P.FLOAT: torch.float32, P.INT64: torch.int64, P.INT32: torch.int32, P.DOUBLE: torch.float64,
          P.BOOL: torch.bool, P.FLOAT16: torch.float16, P.BFLOAT16: torch.bfloat16, P.UINT8: torch.uint8, P.INT8: torch.int8}


class OnnxError(Exception):
    pass


def _parse_tensor(buf: bytes):
    dims, dt, name, raw, floats, ints = [], P.FLOAT, "", None, [], []
    for f, wt, v in P.parse(buf):
        if f == 1: dims += P.packed_ints(v) if wt == 2 else [P.signed(v)]
        elif f == 2: dt = v
        elif f == 8: name = v.decode()
        elif f == 9: raw = v
        elif f == 4: floats += list(struct.unpack(f"<{len(v) // 4}f", v)) if wt == 2 else [struct.unpack("<f", v)[0]]
        elif f == 7: ints += P.packed_ints(v) if wt == 2 else [P.signed(v)]
    if raw is not None:
        arr = np.frombuffer(raw, dtype=_NP[dt]).copy()
    elif floats:
        arr = np.asarray(floats, dtype=np.float32)
    else:
        arr = np.asarray(ints, dtype=np.int64)
    return name, torch.from_numpy(arr.reshape(dims) if dims else arr.reshape(()) if arr.size == 1 else arr)


def _parse_attr(buf: bytes):
    name, val, typ = "", None, 0
    floats, ints = [], []
    for f, wt, v in P.parse(buf):
        if f == 1: name = v.decode()
        elif f == 2: val = struct.unpack("<f", v)[0]
        elif f == 3: val = P.signed(v)
        elif f == 4: val = v.decode(errors="replace")
        elif f == 5: val = _parse_tensor(v)[1]
        elif f == 7: floats += list(struct.unpack(f"<{len(v) // 4}f", v)) if wt == 2 else [struct.unpack("<f", v)[0]]
        elif f == 8: ints += P.packed_ints(v) if wt == 2 else [P.signed(v)]
        elif f == 20: typ = v
    if typ == 6 or (floats and val is None): val = floats
    if typ == 7 or (ints and val is None): val = ints
    return name, val


def _parse_value_info(buf: bytes):
    name, shape = "", []
    for f, _, v in P.parse(buf):
        if f == 1: name = v.decode()
        elif f == 2:
            for f2, _, v2 in P.parse(v):
                if f2 == 1:
                    for f3, _, v3 in P.parse(v2):
                        if f3 == 2:
                            for f4, _, v4 in P.parse(v3):
                                if f4 == 1:
                                    d = None
                                    for f5, _, v5 in P.parse(v4):
                                        d = P.signed(v5) if f5 == 1 else v5.decode()
                                    shape.append(d)
    return name, shape


@dataclasses.dataclass
class ModelInput:
    name: str
    shape: list


@dataclasses.dataclass
class CompiledOp:
    op_type: str
    inputs: list
    outputs: list
    attrs: dict
    name: str = ""


class OnnxModel:
    def __init__(self, ops, inputs, outputs, initializers, name="", opset=17, producer=""):
        self.ops, self.inputs, self.outputs, self.initializers = ops, inputs, outputs, initializers
        self.name, self.opset, self.producer = name, opset, producer

    @classmethod
    def from_proto(cls, data: bytes) -> "OnnxModel":
        graph, opset, producer = None, 17, ""
        for f, _, v in P.parse(data):
            if f == 7: graph = v
            elif f == 2: producer = v.decode()
            elif f == 8:
                for f2, _, v2 in P.parse(v):
                    if f2 == 2: opset = v2
        if graph is None:
            raise OnnxError("ModelProto has no graph")
        ops, inits, ins, outs, gname = [], {}, [], [], ""
        for f, _, v in P.parse(graph):
            if f == 1:
                i, o, a, t, nm = [], [], {}, "", ""
                for f2, _, v2 in P.parse(v):
                    if f2 == 1: i.append(v2.decode())
                    elif f2 == 2: o.append(v2.decode())
                    elif f2 == 3: nm = v2.decode()
                    elif f2 == 4: t = v2.decode()
                    elif f2 == 5:
                        k, val = _parse_attr(v2)
                        a[k] = val
                ops.append(CompiledOp(t, i, o, a, nm))
            elif f == 2: gname = v.decode()
            elif f == 5:
                n, t = _parse_tensor(v)
                inits[n] = t
            elif f == 11: ins.append(ModelInput(*_parse_value_info(v)))
            elif f == 12: outs.append(_parse_value_info(v)[0])
        ins = [i for i in ins if i.name not in inits]
        return cls(ops, ins, outs, inits, gname, opset, producer)

    def get_inputs(self): return self.inputs
    def get_outputs(self): return self.outputs
    def num_parameters(self) -> int: return sum(t.numel() for t in self.initializers.values())

    def to_state_dict(self):
        from ..serialize import StateDict
        return StateDict.from_tensors({k: v.float() for k, v in self.initializers.items() if v.is_floating_point()})

    def forward(self, inputs: dict) -> dict:
        dev = next(iter(inputs.values())).device if inputs else "cpu"
        env = {k: v.to(dev) for k, v in self.initializers.items()}
        env.update(inputs)
        for op in self.ops:
            fn = _OPS.get(op.op_type)
            if fn is None:
                raise OnnxError(f"unsupported operator {op.op_type}")
            res = fn([env[i] if i else None for i in op.inputs], op.attrs)
            res = res if isinstance(res, (tuple, list)) else [res]
            for n, r in zip(op.outputs, res):
                env[n] = r
        return {o: env[o] for o in self.outputs}


def _pool_args(a):
    k, s = a["kernel_shape"], a.get("strides", [1] * len(a["kernel_shape"]))
    p = a.get("pads", [0] * 2 * len(k))
    return tuple(k), tuple(s), tuple(p[: len(k)])


def _axes(x, a, ins, idx=1):
    ax = a.get("axes")
    if ax is None and len(ins) > idx and ins[idx] is not None:
        ax = ins[idx].tolist()
    return tuple(ax) if ax is not None else tuple(range(x.dim()))


_OPS = {
    "Relu": lambda i, a: F.relu(i[0]), "Sigmoid": lambda i, a: torch.sigmoid(i[0]), "Tanh": lambda i, a: torch.tanh(i[0]),
    "Softmax": lambda i, a: torch.softmax(i[0], a.get("axis", -1)), "LeakyRelu": lambda i, a: F.leaky_relu(i[0], a.get("alpha", 0.01)),
    "Gelu": lambda i, a: F.gelu(i[0], approximate="tanh" if a.get("approximate") == "tanh" else "none"),
    "Add": lambda i, a: i[0] + i[1], "Sub": lambda i, a: i[0] - i[1], "Mul": lambda i, a: i[0] * i[1], "Div": lambda i, a: i[0] / i[1],
    "MatMul": lambda i, a: i[0] @ i[1], "Sqrt": lambda i, a: i[0].sqrt(), "Pow": lambda i, a: i[0] ** i[1], "Exp": lambda i, a: i[0].exp(),
    "Log": lambda i, a: i[0].log(), "Neg": lambda i, a: -i[0], "Abs": lambda i, a: i[0].abs(), "Erf": lambda i, a: torch.erf(i[0]),
    "Gemm": lambda i, a: a.get("alpha", 1.0) * ((i[0].t() if a.get("transA") else i[0]) @ (i[1].t() if a.get("transB") else i[1]))
    + (a.get("beta", 1.0) * i[2] if len(i) > 2 and i[2] is not None else 0),
    "Reshape": lambda i, a: i[0].reshape([int(s) if s != 0 else i[0].shape[k] for k, s in enumerate(i[1].tolist())]),
    "Transpose": lambda i, a: i[0].permute(a["perm"]) if "perm" in a else i[0].permute(*reversed(range(i[0].dim()))),
    "Flatten": lambda i, a: i[0].flatten(a.get("axis", 1)) if a.get("axis", 1) else i[0].reshape(1, -1),
    "Squeeze": lambda i, a: (lambda ax: i[0].squeeze() if ax is None else torch.squeeze(i[0], tuple(ax)))(a.get("axes") or (i[1].tolist() if len(i) > 1 and i[1] is not None else None)),
    "Unsqueeze": lambda i, a: (lambda x, ax: [x := x.unsqueeze(d) for d in sorted(ax)][-1])(i[0], a.get("axes") or i[1].tolist()),
    "Concat": lambda i, a: torch.cat(i, a.get("axis", 0)),
    "Gather": lambda i, a: torch.index_select(i[0], a.get("axis", 0), i[1].reshape(-1).long()).reshape(
        i[0].shape[:a.get("axis", 0)] + tuple(i[1].shape) + i[0].shape[a.get("axis", 0) + 1:]),
    "ReduceSum": lambda i, a: i[0].sum(_axes(i[0], a, i), bool(a.get("keepdims", 1))),
    "ReduceMean": lambda i, a: i[0].mean(_axes(i[0], a, i), bool(a.get("keepdims", 1))),
    "ReduceMax": lambda i, a: i[0].amax(_axes(i[0], a, i), bool(a.get("keepdims", 1))),
    "Conv": lambda i, a: F.conv2d(i[0], i[1], i[2] if len(i) > 2 else None, tuple(a.get("strides", [1, 1])),
                                  tuple(a.get("pads", [0, 0, 0, 0])[:2]), tuple(a.get("dilations", [1, 1])), a.get("group", 1)),
    "MaxPool": lambda i, a: F.max_pool2d(i[0], *_pool_args(a)),
    "AveragePool": lambda i, a: F.avg_pool2d(i[0], *_pool_args(a), count_include_pad=bool(a.get("count_include_pad", 0))),
    "GlobalAveragePool": lambda i, a: i[0].mean((-2, -1), keepdim=True),
    "BatchNormalization": lambda i, a: F.batch_norm(i[0], i[3], i[4], i[1], i[2], False, 0.0, a.get("epsilon", 1e-5)),
    "LayerNormalization": lambda i, a: F.layer_norm(i[0], i[0].shape[a.get("axis", -1):], i[1], i[2] if len(i) > 2 else None, a.get("epsilon", 1e-5)),
    "Dropout": lambda i, a: i[0], "Identity": lambda i, a: i[0], "Constant": lambda i, a: a.get("value", torch.tensor(a.get("value_float", a.get("value_int", 0.0)))),
    "Cast": lambda i, a: i[0].to(_TORCH[a["to"]]), "Shape": lambda i, a: torch.tensor(list(i[0].shape), dtype=torch.int64),
    "Equal": lambda i, a: i[0] == i[1], "Greater": lambda i, a: i[0] > i[1], "Less": lambda i, a: i[0] < i[1],
    "Where": lambda i, a: torch.where(i[0].bool(), i[1], i[2]),
    "Clip": lambda i, a: i[0].clamp(a.get("min", i[1].item() if len(i) > 1 and i[1] is not None else None),
                                    a.get("max", i[2].item() if len(i) > 2 and i[2] is not None else None)),
}

SUPPORTED_OPS = sorted(_OPS)


def import_onnx_bytes(data: bytes) -> OnnxModel: return OnnxModel.from_proto(data)


def import_onnx(path) -> OnnxModel:
    with open(path, "rb") as f:
        return OnnxModel.from_proto(f.read())
