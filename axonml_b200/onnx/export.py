"""ONNX export (crates/axonml-onnx/src/export.rs:41-405): ``OnnxExporter`` builder (inputs,
outputs, nodes with attributes, initializers), opset 17, ``export_feedforward`` for Linear/activation
stacks and ``export_module`` for ``Sequential`` models made of the supported layers."""
from __future__ import annotations

import numpy as np
import torch

from . import proto as P

OPSET = 17


def _tensor(name: str, arr: np.ndarray) -> bytes:
    dt = {np.dtype("float32"): P.FLOAT, np.dtype("int64"): P.INT64}[arr.dtype]
    b = b"".join(P.enc_varint(1, int(d)) for d in arr.shape) + P.enc_varint(2, dt) + P.enc_str(8, name)
    return b + P.enc_bytes(9, arr.astype(arr.dtype.newbyteorder("<")).tobytes())


def _value_info(name: str, shape, dtype: int = P.FLOAT) -> bytes:
    dims = b""
    for d in shape:
        dims += P.enc_bytes(1, P.enc_str(2, d) if isinstance(d, str) else P.enc_varint(1, int(d)))
    tt = P.enc_varint(1, dtype) + P.enc_bytes(2, dims)
    return P.enc_str(1, name) + P.enc_bytes(2, P.enc_bytes(1, tt))


def _attr(name: str, v) -> bytes:
    b = P.enc_str(1, name)
    if isinstance(v, bool) or isinstance(v, int): return b + P.enc_varint(3, int(v)) + P.enc_varint(20, 2)
    if isinstance(v, float): return b + P.enc_float(2, v) + P.enc_varint(20, 1)
    if isinstance(v, str): return b + P.enc_bytes(4, v.encode()) + P.enc_varint(20, 3)
    if isinstance(v, (list, tuple)) and all(isinstance(x, int) for x in v):
        return b + b"".join(P.enc_varint(8, x) for x in v) + P.enc_varint(20, 7)
    if isinstance(v, (list, tuple)): return b + b"".join(P.enc_float(7, float(x)) for x in v) + P.enc_varint(20, 6)
    if isinstance(v, np.ndarray): return b + P.enc_bytes(5, _tensor("", v)) + P.enc_varint(20, 4)
    raise TypeError(f"unsupported attribute {name}={v!r}")


class OnnxExporter:
    def __init__(self, name: str):
        self.name, self.producer, self.version, self.doc = name, "axonml_b200", "0.1.0", ""
        self.inputs, self.outputs, self.nodes, self.inits = [], [], [], []

    @classmethod
    def new(cls, name): return cls(name)
    def with_producer(self, name, version): self.producer, self.version = name, version; return self
    def with_doc_string(self, doc): self.doc = doc; return self
    def add_input(self, name, shape, dtype=P.FLOAT): self.inputs.append((name, list(shape), dtype))
    def add_output(self, name, shape, dtype=P.FLOAT): self.outputs.append((name, list(shape), dtype))

    def add_node(self, op_type, inputs, outputs, attrs=None, name=None):
        self.nodes.append((op_type, list(inputs), list(outputs), dict(attrs or {}), name or f"{op_type}_{len(self.nodes)}"))

    def add_named_node(self, name, op_type, inputs, outputs, attrs=None): self.add_node(op_type, inputs, outputs, attrs, name)
    def add_initializer(self, name, tensor: torch.Tensor): self.inits.append((name, tensor.detach().cpu().float().numpy()))
    def add_initializer_data(self, name, shape, data): self.inits.append((name, np.asarray(data, dtype=np.float32).reshape(shape)))
    def add_int64_initializer(self, name, data): self.inits.append((name, np.asarray(data, dtype=np.int64)))

    def to_bytes(self) -> bytes:
        g = b""
        for op, ins, outs, attrs, nm in self.nodes:
            n = b"".join(P.enc_str(1, i) for i in ins) + b"".join(P.enc_str(2, o) for o in outs)
            n += P.enc_str(3, nm) + P.enc_str(4, op) + b"".join(P.enc_bytes(5, _attr(k, v)) for k, v in attrs.items())
            g += P.enc_bytes(1, n)
        g += P.enc_str(2, self.name)
        g += b"".join(P.enc_bytes(5, _tensor(n, a)) for n, a in self.inits)
        g += b"".join(P.enc_bytes(11, _value_info(*i)) for i in self.inputs)
        g += b"".join(P.enc_bytes(12, _value_info(*o)) for o in self.outputs)
        m = P.enc_varint(1, 8) + P.enc_str(2, self.producer) + P.enc_str(3, self.version)
        if self.doc:
            m += P.enc_str(6, self.doc)
        m += P.enc_bytes(7, g) + P.enc_bytes(8, P.enc_str(1, "") + P.enc_varint(2, OPSET))
        return m

    def to_proto(self):
        """The model as a ``ModelProto`` message object (export.rs: ``OnnxExporter::to_proto``)."""
        from .messages import ModelProto
        return ModelProto.from_bytes(self.to_bytes())

    def export(self, path) -> None:
        with open(path, "wb") as f:
            f.write(self.to_bytes())


def export_onnx(exporter: OnnxExporter, path) -> None: exporter.export(path)
def export_onnx_bytes(exporter: OnnxExporter) -> bytes: return exporter.to_bytes()


def export_feedforward(name: str, layers, input_size: int, activation: str = "Relu") -> OnnxExporter:
    """``layers``: list of (weight[out,in], bias[out]) tensors -> Gemm(+activation) chain."""
    ex = OnnxExporter(name)
    ex.add_input("input", ["batch", input_size])
    cur = "input"
    for i, (w, b) in enumerate(layers):
        ex.add_initializer(f"fc{i}.weight", w)
        ex.add_initializer(f"fc{i}.bias", b)
        out = f"fc{i}_out"
        ex.add_node("Gemm", [cur, f"fc{i}.weight", f"fc{i}.bias"], [out], {"transB": 1, "alpha": 1.0, "beta": 1.0})
        cur = out
        if i + 1 < len(layers) and activation:
            ex.add_node(activation, [cur], [f"act{i}_out"])
            cur = f"act{i}_out"
    ex.add_node("Identity", [cur], ["output"])
    ex.add_output("output", ["batch", layers[-1][0].shape[0]])
    return ex


def export_module(module, input_shape, name: str = "model") -> OnnxExporter:
    """Exports a ``Sequential`` of Linear / Conv2d / BatchNorm2d / pooling / activation / Flatten /
    Dropout layers."""
    from .. import nn
    ex = OnnxExporter(name)
    ex.add_input("input", ["batch"] + list(input_shape[1:]))
    cur, k = "input", 0
    act = {nn.ReLU: "Relu", nn.Sigmoid: "Sigmoid", nn.Tanh: "Tanh", nn.GELU: "Gelu", nn.Identity: "Identity"}
    if not isinstance(module, nn.Sequential):
        # a wrapper whose only child is the layer stack (MLP), or whose children run in order
        subs = list(module.children())
        module = subs[0] if len(subs) == 1 and isinstance(subs[0], nn.Sequential) else subs
    for layer in module:
        out = f"t{k}"
        k += 1
        if isinstance(layer, nn.Linear):
            ex.add_initializer(f"{out}.weight", layer.weight)
            ins = [cur, f"{out}.weight"]
            if layer.bias is not None:
                ex.add_initializer(f"{out}.bias", layer.bias)
                ins.append(f"{out}.bias")
            ex.add_node("Gemm", ins, [out], {"transB": 1})
        elif isinstance(layer, nn.Conv2d):
            ex.add_initializer(f"{out}.weight", layer.weight)
            ins = [cur, f"{out}.weight"]
            if layer.bias is not None:
                ex.add_initializer(f"{out}.bias", layer.bias)
                ins.append(f"{out}.bias")
            ph, pw = layer.padding
            ex.add_node("Conv", ins, [out], {"kernel_shape": list(layer.kernel_size), "strides": list(layer.stride), "pads": [ph, pw, ph, pw]})
        elif isinstance(layer, nn.BatchNorm2d):
            for nm, t in (("scale", layer.weight), ("B", layer.bias), ("mean", layer.running_mean), ("var", layer.running_var)):
                ex.add_initializer(f"{out}.{nm}", t)
            ex.add_node("BatchNormalization", [cur] + [f"{out}.{n}" for n in ("scale", "B", "mean", "var")], [out], {"epsilon": float(layer.eps)})
        elif isinstance(layer, (nn.MaxPool2d, nn.AvgPool2d)):
            ks = layer.kernel_size if isinstance(layer.kernel_size, (tuple, list)) else (layer.kernel_size,) * 2
            st = layer.stride if isinstance(layer.stride, (tuple, list)) else (layer.stride,) * 2
            p = layer.padding if isinstance(layer.padding, (tuple, list)) else (layer.padding,) * 2
            ex.add_node("MaxPool" if isinstance(layer, nn.MaxPool2d) else "AveragePool", [cur], [out],
                        {"kernel_shape": list(ks), "strides": list(st), "pads": [p[0], p[1], p[0], p[1]]})
        elif isinstance(layer, nn.Dropout):
            ex.add_node("Dropout", [cur], [out])
        elif isinstance(layer, nn.Softmax):
            ex.add_node("Softmax", [cur], [out], {"axis": layer.dim})
        elif type(layer) in act:
            ex.add_node(act[type(layer)], [cur], [out])
        elif isinstance(layer, torch.nn.Flatten):
            ex.add_node("Flatten", [cur], [out], {"axis": 1})
        else:
            raise NotImplementedError(f"cannot export {type(layer).__name__}")
        cur = out
    ex.add_node("Identity", [cur], ["output"])
    ex.add_output("output", ["batch", -1])
    return ex
