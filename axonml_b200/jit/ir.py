"""JIT intermediate representation (crates/axonml-jit/src/ir.rs:139-262): a flat SSA graph of
``Node{id, op, dtype, shape}``.  ``Op`` carries the reference's 41 operation kinds by name."""
from __future__ import annotations

import dataclasses
import enum

from .error import InvalidGraph, UnsupportedOp


class NodeId(int):
    """Index of a node in its graph (ir.rs:8-16); an ``int`` with the reference's ``index()``."""

    def index(self) -> int:
        return int(self)

    def __repr__(self) -> str:
        return f"%{int(self)}"


class Shape(tuple):
    """Static shape of a traced value (ir.rs:52-110)."""

    def __new__(cls, dims=()):
        return super().__new__(cls, (int(d) for d in dims))

    @classmethod
    def new(cls, dims): return cls(dims)

    def dims(self) -> tuple: return tuple(self)
    def ndim(self) -> int: return len(self)

    def numel(self) -> int:
        n = 1
        for d in self:
            n *= d
        return n

    def broadcast_compatible(self, other) -> bool:
        other = tuple(other)
        for i in range(max(len(self), len(other))):
            a = self[len(self) - 1 - i] if i < len(self) else 1
            b = other[len(other) - 1 - i] if i < len(other) else 1
            if a != b and a != 1 and b != 1:
                return False
        return True

    def broadcast_shape(self, other):
        """The common shape, or ``None`` when the two do not broadcast."""
        if not self.broadcast_compatible(other):
            return None
        other = tuple(other)
        out = []
        for i in range(max(len(self), len(other))):
            a = self[len(self) - 1 - i] if i < len(self) else 1
            b = other[len(other) - 1 - i] if i < len(other) else 1
            out.append(max(a, b) if 0 not in (a, b) else 0)
        return Shape(reversed(out))


class DataType(enum.Enum):
    F32 = "f32"
    F64 = "f64"
    I32 = "i32"
    I64 = "i64"
    Bool = "bool"

    def size_bytes(self) -> int:
        return {"f32": 4, "i32": 4, "f64": 8, "i64": 8, "bool": 1}[self.value]


UNARY = ("Neg", "Abs", "Sqrt", "Exp", "Log", "Sin", "Cos", "Tanh", "Relu", "Sigmoid", "Gelu", "Silu", "Contiguous")
BINARY = ("Add", "Sub", "Mul", "Div", "Pow", "Max", "Min", "Gt", "Lt", "Eq")
SCALAR = ("AddScalar", "MulScalar")
REDUCE = ("Sum", "Mean", "SumAxis", "MeanAxis", "MaxAxis")
SHAPE = ("Reshape", "Transpose", "Squeeze", "Unsqueeze", "Broadcast")
OTHER = ("Input", "Output", "Constant", "MatMul", "Where", "Cast")
ALL_OPS = UNARY + BINARY + SCALAR + REDUCE + SHAPE + OTHER
ELEMENTWISE = set(UNARY + BINARY + SCALAR + ("Where", "Cast", "Constant"))


@dataclasses.dataclass(frozen=True)
class Op:
    kind: str
    inputs: tuple = ()
    attrs: tuple = ()          # sorted (key, value) pairs

    def attr(self, key, default=None):
        for k, v in self.attrs:
            if k == key:
                return v
        return default

    @staticmethod
    def make(kind: str, inputs=(), **attrs) -> "Op":
        if kind not in ALL_OPS:
            raise UnsupportedOp(kind)
        norm = tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in attrs.items()))
        return Op(kind, tuple(inputs), norm)

    def is_elementwise(self) -> bool: return self.kind in ELEMENTWISE
    def is_reduction(self) -> bool: return self.kind in REDUCE


@dataclasses.dataclass
class Node:
    id: int
    op: Op
    dtype: DataType
    shape: tuple


class Graph:
    def __init__(self):
        self.nodes: list[Node] = []
        self.inputs: dict[str, int] = {}
        self.outputs: dict[str, int] = {}

    @classmethod
    def new(cls): return cls()

    def add_node(self, op: Op, dtype: DataType, shape) -> int:
        nid = NodeId(len(self.nodes))
        self.nodes.append(Node(nid, op, dtype, Shape(shape)))
        if op.kind == "Input":
            self.inputs[op.attr("name")] = nid
        if op.kind == "Output":
            self.outputs[op.attr("name")] = nid
        return nid

    def register_input(self, name: str, nid: int) -> None:
        """Names node ``nid`` as the graph input ``name`` (``add_node`` does this for Input nodes)."""
        self.inputs[name] = NodeId(nid)

    def register_output(self, name: str, nid: int) -> None:
        self.outputs[name] = NodeId(nid)

    def input(self, name: str): return self.inputs.get(name)
    def output(self, name: str): return self.outputs.get(name)
    def node_mut(self, nid: int) -> Node: return self.nodes[nid]          # nodes are mutable objects

    def topological_order(self) -> list:
        """Node ids with every node after its inputs: nodes can only refer to earlier ones, so
        this is the order of insertion."""
        return [n.id for n in self.nodes]

    def node(self, nid: int) -> Node: return self.nodes[nid]
    def len(self) -> int: return len(self.nodes)
    def __len__(self) -> int: return len(self.nodes)
    def is_empty(self) -> bool: return not self.nodes
    def input_names(self): return list(self.inputs)
    def output_names(self): return list(self.outputs)

    def users(self) -> dict:
        u: dict = {n.id: [] for n in self.nodes}
        for n in self.nodes:
            for i in n.op.inputs:
                u[i].append(n.id)
        return u

    def validate(self) -> None:
        for n in self.nodes:
            for i in n.op.inputs:
                if not 0 <= i < n.id:
                    raise InvalidGraph(f"node {n.id} uses {i} before its definition")

    def signature(self) -> tuple:
        return tuple((n.op.kind, n.op.inputs, n.op.attrs, n.dtype.value, n.shape) for n in self.nodes)

    def __repr__(self) -> str:
        return "\n".join(f"%{n.id} = {n.op.kind}{list(n.op.inputs)} {dict(n.op.attrs)} : {n.dtype.value}{list(n.shape)}" for n in self.nodes)
