"""Graph tracing (crates/axonml-jit/src/trace.rs:595-630): ``trace(lambda t: ...)`` hands the
closure a ``Tracer``; ``t.input(name, shape)`` returns a ``TracedValue`` whose methods append nodes."""
from __future__ import annotations

from .ir import DataType, Graph, Op
from ..tensor.view import broadcast_shape


class TracedValue:
    def __init__(self, tracer: "Tracer", nid: int):
        self.tracer, self.id = tracer, nid

    def node_id(self) -> int: return self.id
    @property
    def shape(self): return self.tracer.graph.node(self.id).shape

    def _bin(self, kind, other):
        if not isinstance(other, TracedValue):
            other = self.tracer.constant(float(other))
        g = self.tracer.graph
        shape = broadcast_shape(list(self.shape), list(other.shape))
        dt = DataType.Bool if kind in ("Gt", "Lt", "Eq") else g.node(self.id).dtype
        return TracedValue(self.tracer, g.add_node(Op.make(kind, (self.id, other.id)), dt, shape))

    def _un(self, kind, **attrs):
        g = self.tracer.graph
        return TracedValue(self.tracer, g.add_node(Op.make(kind, (self.id,), **attrs), g.node(self.id).dtype, self.shape))

    def add(self, o): return self._bin("Add", o)
    def sub(self, o): return self._bin("Sub", o)
    def mul(self, o): return self._bin("Mul", o)
    def div(self, o): return self._bin("Div", o)
    def pow(self, o): return self._bin("Pow", o)
    def max(self, o): return self._bin("Max", o)
    def min(self, o): return self._bin("Min", o)
    def gt(self, o): return self._bin("Gt", o)
    def lt(self, o): return self._bin("Lt", o)
    def eq(self, o): return self._bin("Eq", o)
    __add__, __sub__, __mul__, __truediv__ = add, sub, mul, div
    def add_scalar(self, s): return self._un("AddScalar", scalar=float(s))
    def mul_scalar(self, s): return self._un("MulScalar", scalar=float(s))
    def neg(self): return self._un("Neg")
    def abs(self): return self._un("Abs")
    def sqrt(self): return self._un("Sqrt")
    def exp(self): return self._un("Exp")
    def log(self): return self._un("Log")
    def sin(self): return self._un("Sin")
    def cos(self): return self._un("Cos")
    def tanh(self): return self._un("Tanh")
    def relu(self): return self._un("Relu")
    def sigmoid(self): return self._un("Sigmoid")
    def gelu(self): return self._un("Gelu")
    def silu(self): return self._un("Silu")
    def contiguous(self): return self._un("Contiguous")

    def _shape_op(self, kind, out_shape, **attrs):
        g = self.tracer.graph
        return TracedValue(self.tracer, g.add_node(Op.make(kind, (self.id,), **attrs), g.node(self.id).dtype, out_shape))

    def sum(self): return self._shape_op("Sum", ())
    def mean(self): return self._shape_op("Mean", ())

    def _axis(self, kind, axis, keepdim):
        s = list(self.shape)
        a = axis % len(s)
        out = s[:a] + ([1] if keepdim else []) + s[a + 1:]
        return self._shape_op(kind, out, axis=a, keepdim=bool(keepdim))

    def sum_axis(self, axis, keepdim=False): return self._axis("SumAxis", axis, keepdim)
    def mean_axis(self, axis, keepdim=False): return self._axis("MeanAxis", axis, keepdim)
    def max_axis(self, axis, keepdim=False): return self._axis("MaxAxis", axis, keepdim)

    def reshape(self, shape):
        from ..tensor.view import reshape_infer
        return self._shape_op("Reshape", reshape_infer(list(self.shape), list(shape)), shape=tuple(shape))

    def transpose(self, d0, d1):
        s = list(self.shape)
        s[d0], s[d1] = s[d1], s[d0]
        return self._shape_op("Transpose", s, dim0=d0, dim1=d1)

    def squeeze(self, dim):
        s = list(self.shape)
        s.pop(dim)
        return self._shape_op("Squeeze", s, dim=dim)

    def unsqueeze(self, dim):
        s = list(self.shape)
        s.insert(dim if dim >= 0 else len(s) + 1 + dim, 1)
        return self._shape_op("Unsqueeze", s, dim=dim)

    def broadcast(self, shape): return self._shape_op("Broadcast", list(shape), shape=tuple(shape))

    def matmul(self, o):
        a, b = list(self.shape), list(o.shape)
        shape = a[:-1] + b[-1:]
        g = self.tracer.graph
        return TracedValue(self.tracer, g.add_node(Op.make("MatMul", (self.id, o.id)), g.node(self.id).dtype, shape))

    def where(self, cond, other):
        g = self.tracer.graph
        return TracedValue(self.tracer, g.add_node(Op.make("Where", (cond.id, self.id, other.id)), g.node(self.id).dtype, self.shape))

    def cast(self, dtype: DataType):
        return TracedValue(self.tracer, self.tracer.graph.add_node(Op.make("Cast", (self.id,), dtype=dtype.value), dtype, self.shape))


class Tracer:
    def __init__(self):
        self.graph = Graph()

    def input(self, name: str, shape, dtype: DataType = DataType.F32) -> TracedValue:
        return TracedValue(self, self.graph.add_node(Op.make("Input", (), name=name), dtype, shape))

    def constant(self, value: float) -> TracedValue:
        return TracedValue(self, self.graph.add_node(Op.make("Constant", (), value=float(value)), DataType.F32, ()))

    def output(self, name: str, value: TracedValue) -> TracedValue:
        n = self.graph.node(value.id)
        return TracedValue(self, self.graph.add_node(Op.make("Output", (value.id,), name=name), n.dtype, n.shape))


def trace(fn) -> Graph:
    t = Tracer()
    fn(t)
    t.graph.validate()
    return t.graph
