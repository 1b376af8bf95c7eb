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


class FusionError(Exception):
    """Errors of the fusion package (crates/axonml-fusion/src/error.rs:15-40), one subclass per variant."""


class ShapeMismatch(FusionError, ValueError):
    def __init__(self, expected, actual):
        super().__init__(f"Invalid input shape: expected {list(expected)}, got {list(actual)}")
        self.expected, self.actual = list(expected), list(actual)


class NotFusable(FusionError):
    def __init__(self, what): super().__init__(f"Pattern not fusable: {what}")


class InvalidConfig(FusionError, ValueError):
    def __init__(self, what): super().__init__(f"Invalid fusion configuration: {what}")


class ExecutionError(FusionError, RuntimeError):
    def __init__(self, what): super().__init__(f"Execution error: {what}")


class TensorError(FusionError):
    def __init__(self, what): super().__init__(f"Tensor conversion error: {what}")


class FusedOp:
    def execute(self, x: torch.Tensor) -> torch.Tensor: raise NotImplementedError
    def forward(self, x: torch.Tensor) -> torch.Tensor: return self.execute(x)
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
        if weight.dim() != 2:
            raise InvalidConfig(f"weight must be [out_features, in_features], got {list(weight.shape)}")
        if bias is not None and tuple(bias.shape) != (weight.shape[0],):
            raise ShapeMismatch([weight.shape[0]], bias.shape)
        self.weight, self.bias = weight, bias
        try:
            self.activation = activation if isinstance(activation, Activation) else Activation(activation or "none")
        except ValueError as e:
            raise InvalidConfig(f"unknown activation {activation!r}") from e

    @classmethod
    def new(cls, weight, bias=None, activation=Activation.None_): return cls(weight, bias, activation)

    def execute(self, x):
        if x.shape[-1] != self.weight.shape[1]:
            raise ShapeMismatch([self.weight.shape[1]], [x.shape[-1]])
        return linear(x, self.weight, self.bias, self.activation.value)

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

    def apply(self, x, *args):
        """The operation on a number or a tensor; ``args`` are its constants (the addend, the
        factor, the slope, the clamp bounds)."""
        t = torch.is_tensor(x)
        v = x if t else torch.tensor(float(x))
        k = self.value
        if k == "add": r = v + args[0]
        elif k == "mul": r = v * args[0]
        elif k == "relu": r = v.clamp_min(0)
        elif k == "leaky_relu": r = torch.where(v > 0, v, v * (args[0] if args else 0.01))
        elif k == "sigmoid": r = torch.sigmoid(v)
        elif k == "tanh": r = torch.tanh(v)
        elif k == "exp": r = torch.exp(v)
        elif k == "log": r = torch.log(v)
        elif k == "sqrt": r = torch.sqrt(v)
        elif k == "square": r = v * v
        elif k == "clamp": r = v.clamp(args[0], args[1])
        elif k == "neg": r = -v
        else: r = v.abs()
        return r if t else float(r)


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


# convenience constructors (crates/axonml-fusion/src/linear.rs:206-224, elementwise.rs:241-262)
def fuse_matmul_bias_relu(weight, bias) -> FusedLinear: return FusedLinear(weight, bias, Activation.Relu)
def fuse_matmul_bias_gelu(weight, bias) -> FusedLinear: return FusedLinear(weight, bias, Activation.Gelu)
def fuse_matmul_bias(weight, bias) -> FusedLinear: return FusedLinear(weight, bias, Activation.None_)


def fuse_elementwise(ops) -> FusedElementwise:
    """Chain from a list of steps: ``ElementwiseOp`` members for the argument-free ones, ``(op,
    arg, ...)`` tuples for Add / Mul / LeakyRelu / Clamp."""
    steps = []
    for o in ops:
        op, args = (o[0], tuple(float(a) for a in o[1:])) if isinstance(o, (tuple, list)) else (o, ())
        if not isinstance(op, ElementwiseOp):
            raise InvalidConfig(f"{op!r} is not an ElementwiseOp")
        steps.append((op, args))
    return FusedElementwise(steps)


def fused_add_relu(bias: float) -> FusedElementwise: return FusedElementwise.builder().add(bias).relu().build()
def fused_mul_add(scale: float, bias: float) -> FusedElementwise: return FusedElementwise.builder().mul(scale).add(bias).build()


def fused_scale_bias_relu(scale: float, bias: float) -> FusedElementwise:
    return FusedElementwise.builder().mul(scale).add(bias).relu().build()
