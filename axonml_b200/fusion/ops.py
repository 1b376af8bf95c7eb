"""Fused operators (crates/axonml-fusion/src/lib.rs:48-60, linear.rs:20-175,
elementwise.rs:20-256): the ``FusedOp`` protocol, ``FusedLinear`` = act(x W^T + b) in one pass
(tcgen05 GEMM with the bias/activation epilogue on a B200) and the ``FusedElementwise`` chain
builder, which on CUDA compiles the whole chain into one NVRTC-generated kernel."""
from __future__ import annotations

import enum

import torch

from ..jit.ir import DataType
from ..jit.trace import Tracer
from ..ops.linear import linear


class FusedOp:
    def execute(self, x: torch.Tensor) -> torch.Tensor: raise NotImplementedError
    def name(self) -> str: return type(self).__name__
    def num_ops(self) -> int: return 1
    def __call__(self, x): return self.execute(x)


class Activation(enum.Enum):
    None_ = "none"
    Relu = "relu"
    Gelu = "gelu"
    Sigmoid = "sigmoid"
    Tanh = "tanh"
    Silu = "silu"


class FusedLinear(FusedOp):
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, activation=Activation.None_):
        self.weight, self.bias = weight, bias
        self.activation = activation if isinstance(activation, Activation) else Activation(activation or "none")

    @classmethod
    def new(cls, weight, bias=None, activation=Activation.None_): return cls(weight, bias, activation)

    def execute(self, x): return linear(x, self.weight, self.bias, self.activation.value)
    def num_ops(self) -> int: return 1 + (self.bias is not None) + (self.activation is not Activation.None_)
    def name(self) -> str: return f"FusedLinear[{self.activation.value}]"


class ElementwiseOp(enum.Enum):
    Add = "add"
    Mul = "mul"
    Relu = "relu"
    LeakyRelu = "leaky_relu"
    Sigmoid = "sigmoid"
    Tanh = "tanh"
    Exp = "exp"
    Log = "log"
    Sqrt = "sqrt"
    Square = "square"
    Clamp = "clamp"
    Neg = "neg"
    Abs = "abs"


class FusedElementwise(FusedOp):
    """Chain of unary elementwise steps with scalar operands, e.g.
    ``FusedElementwise.builder().mul(2.0).add(1.0).relu().build()``."""

    def __init__(self, steps):
        self.steps = list(steps)
        self._compiled = None

    @staticmethod
    def builder() -> "FusedElementwiseBuilder": return FusedElementwiseBuilder()

    def num_ops(self) -> int: return len(self.steps)
    def name(self) -> str: return "FusedElementwise[" + ",".join(op.value for op, _ in self.steps) + "]"

    def _graph(self, shape):
        t = Tracer()
        v = t.input("x", list(shape), DataType.F32)
        for op, args in self.steps:
            if op is ElementwiseOp.Add: v = v.add_scalar(args[0])
            elif op is ElementwiseOp.Mul: v = v.mul_scalar(args[0])
            elif op is ElementwiseOp.Relu: v = v.relu()
            elif op is ElementwiseOp.LeakyRelu: v = v.max(v.mul_scalar(args[0]))
            elif op is ElementwiseOp.Sigmoid: v = v.sigmoid()
            elif op is ElementwiseOp.Tanh: v = v.tanh()
            elif op is ElementwiseOp.Exp: v = v.exp()
            elif op is ElementwiseOp.Log: v = v.log()
            elif op is ElementwiseOp.Sqrt: v = v.sqrt()
            elif op is ElementwiseOp.Square: v = v.mul(v)
            elif op is ElementwiseOp.Clamp: v = v.max(t.constant(args[0])).min(t.constant(args[1]))
            elif op is ElementwiseOp.Neg: v = v.neg()
            elif op is ElementwiseOp.Abs: v = v.abs()
        t.output("y", v)
        return t.graph

    def execute(self, x):
        from ..jit.codegen import CompiledFunction
        key = (tuple(x.shape), x.device.type)
        if self._compiled is None or self._compiled[0] != key:
            self._compiled = (key, CompiledFunction(self._graph(x.shape)))
        xin = x if x.dtype == torch.float32 else x.float()
        return self._compiled[1].run_tensors({"x": xin})["y"].to(x.dtype)


class FusedElementwiseBuilder:
    def __init__(self): self._steps = []
    def _push(self, op, *args): self._steps.append((op, args)); return self
    def add(self, c: float): return self._push(ElementwiseOp.Add, float(c))
    def mul(self, c: float): return self._push(ElementwiseOp.Mul, float(c))
    def relu(self): return self._push(ElementwiseOp.Relu)
    def leaky_relu(self, slope: float = 0.01): return self._push(ElementwiseOp.LeakyRelu, float(slope))
    def sigmoid(self): return self._push(ElementwiseOp.Sigmoid)
    def tanh(self): return self._push(ElementwiseOp.Tanh)
    def exp(self): return self._push(ElementwiseOp.Exp)
    def log(self): return self._push(ElementwiseOp.Log)
    def sqrt(self): return self._push(ElementwiseOp.Sqrt)
    def square(self): return self._push(ElementwiseOp.Square)
    def clamp(self, lo: float, hi: float): return self._push(ElementwiseOp.Clamp, float(lo), float(hi))
    def neg(self): return self._push(ElementwiseOp.Neg)
    def abs(self): return self._push(ElementwiseOp.Abs)
    def build(self) -> FusedElementwise: return FusedElementwise(self._steps)


def fuse_linear(weight, bias=None, activation=Activation.None_) -> FusedLinear:
    return FusedLinear(weight, bias, activation)


def fused_elementwise() -> FusedElementwiseBuilder:
    return FusedElementwiseBuilder()
