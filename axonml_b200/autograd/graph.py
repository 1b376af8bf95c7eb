"""Views of the recorded computation graph and user-defined gradient functions.

Parity: crates/axonml-autograd/src/grad_fn.rs:25-100 (``GradientFunction`` with ``apply(grad_output)
-> one gradient (or None) per input``, ``name``, ``next_functions``; ``GradFn`` = shared handle with
``apply`` / ``name`` / ``next_functions`` / ``id``) and src/graph.rs:35-160 (``GraphNode{id, grad_fn,
requires_grad, is_leaf, topo_order}``, ``ComputationGraph`` with ``len`` / ``is_empty`` /
``get_node`` / ``clear``).  The tape itself is torch's; ``GradFn`` wraps one of its nodes,
``ComputationGraph.from_output`` walks the nodes an output depends on, and a ``GradientFunction``
subclass is how a user supplies the backward of an operation written outside the tape."""
from __future__ import annotations

import dataclasses

import torch


class GradFn:
    """Handle on one backward node of the tape."""

    def __init__(self, node):
        self.node = node

    def apply(self, *grad_outputs):
        """Gradients with respect to the node's inputs (a tuple; ``None`` where an input needs none)."""
        out = self.node(*grad_outputs)
        return out if isinstance(out, tuple) else (out,)

    def name(self) -> str:
        return self.node.name()

    def next_functions(self) -> list:
        return [GradFn(fn) if fn is not None else None for fn, _ in self.node.next_functions]

    def id(self) -> int:
        return id(self.node)

    def is_accumulate_grad(self) -> bool:
        return self.name().endswith("AccumulateGrad")

    def __eq__(self, other) -> bool:
        return isinstance(other, GradFn) and other.node is self.node

    def __hash__(self) -> int:
        return id(self.node)

    def __repr__(self) -> str:
        return f"GradFn({self.name()})"


@dataclasses.dataclass
class GraphNode:
    id: int
    grad_fn: GradFn | None
    requires_grad: bool
    is_leaf: bool
    topo_order: int              # 0 for leaves; an operation's is one more than the largest among its inputs

    @classmethod
    def leaf(cls, requires_grad: bool, node_id: int = 0):
        return cls(node_id, None, requires_grad, True, 0)

    @classmethod
    def intermediate(cls, grad_fn: GradFn, requires_grad: bool, topo_order: int, node_id: int = 0):
        return cls(node_id, grad_fn, requires_grad, False, topo_order)


class ComputationGraph:
    """The nodes an output was computed from, leaves first."""

    def __init__(self):
        self._nodes: dict[int, GraphNode] = {}
        self._next_id = 0

    @classmethod
    def new(cls): return cls()

    def _add(self, node: GraphNode) -> GraphNode:
        node.id = self._next_id
        self._next_id += 1
        self._nodes[node.id] = node
        return node

    def register_leaf(self, requires_grad: bool) -> GraphNode:
        return self._add(GraphNode.leaf(requires_grad))

    def register_operation(self, grad_fn: GradFn, requires_grad: bool, topo_order: int | None = None) -> GraphNode:
        order = topo_order if topo_order is not None else 1 + max((n.topo_order for n in self._nodes.values()), default=0)
        return self._add(GraphNode.intermediate(grad_fn, requires_grad, order))

    @classmethod
    def from_output(cls, output: torch.Tensor):
        """Graph of everything ``output`` depends on.  Leaves are the tensors gradients accumulate
        into (parameters and inputs with ``requires_grad``)."""
        g = cls()
        if output.grad_fn is None:
            g.register_leaf(output.requires_grad)
            return g
        order: dict = {}
        post = []
        stack = [(output.grad_fn, False)]
        seen = set()
        while stack:                                          # iterative post-order: inputs before users
            fn, done = stack.pop()
            if done:
                post.append(fn)
                continue
            if fn in seen:
                continue
            seen.add(fn)
            stack.append((fn, True))
            for nxt, _ in fn.next_functions:
                if nxt is not None and nxt not in seen:
                    stack.append((nxt, False))
        for fn in post:
            h = GradFn(fn)
            if h.is_accumulate_grad():
                order[fn] = 0
                n = g.register_leaf(True)
                n.grad_fn = h
            else:
                order[fn] = 1 + max((order[nxt] for nxt, _ in fn.next_functions if nxt is not None), default=0)
                g.register_operation(h, True, order[fn])
        return g

    def get_node(self, node_id: int): return self._nodes.get(node_id)
    def nodes(self) -> list: return list(self._nodes.values())
    def leaves(self) -> list: return [n for n in self._nodes.values() if n.is_leaf]
    def operations(self) -> list: return [n for n in self._nodes.values() if not n.is_leaf]
    def len(self) -> int: return len(self._nodes)
    def __len__(self) -> int: return len(self._nodes)
    def is_empty(self) -> bool: return not self._nodes
    def depth(self) -> int: return max((n.topo_order for n in self._nodes.values()), default=0)

    def clear(self) -> None:
        self._nodes.clear()
        self._next_id = 0

    def reset_id_counter(self) -> None:
        """Node ids start again from 0 for nodes registered from now on (ids are per graph here)."""
        self._next_id = 0

    def op_counts(self) -> dict:
        out: dict[str, int] = {}
        for n in self.operations():
            out[n.grad_fn.name()] = out.get(n.grad_fn.name(), 0) + 1
        return out

    def to_dot(self) -> str:
        """Graphviz text of the graph (edges point from an operation to what it differentiates into)."""
        by_fn = {n.grad_fn: n for n in self._nodes.values() if n.grad_fn is not None}
        lines = ["digraph autograd {"]
        for n in self._nodes.values():
            label = "leaf" if n.grad_fn is None else n.grad_fn.name()
            lines.append(f'  n{n.id} [label="{label}"{", shape=box" if n.is_leaf else ""}];')
        for n in self._nodes.values():
            if n.grad_fn is None or n.is_leaf:
                continue
            for nxt in n.grad_fn.next_functions():
                if nxt is not None and nxt in by_fn:
                    lines.append(f"  n{n.id} -> n{by_fn[nxt].id};")
        lines.append("}")
        return "\n".join(lines)


class GradientFunction:
    """Base class for an operation with a hand-written backward.

    Subclasses implement ``forward(*inputs)`` (may stash tensors on ``self`` or call
    ``self.save_for_backward``) and ``apply(grad_output)`` returning one gradient (or ``None``) per
    input.  ``MyFn.call(*inputs)`` runs the forward outside the tape and records a node whose
    backward is ``apply``."""

    def name(self) -> str:
        return type(self).__name__

    def save_for_backward(self, *tensors) -> None:
        self.saved_tensors = tensors

    def forward(self, *inputs):
        raise NotImplementedError

    def apply(self, grad_output):
        raise NotImplementedError

    @classmethod
    def call(cls, *inputs, **kwargs):
        inst = cls(**kwargs)
        return _Bridge.apply(inst, *inputs)


class _Bridge(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inst, *inputs):
        ctx.inst, ctx.n = inst, len(inputs)
        with torch.no_grad():
            return inst.forward(*inputs)

    @staticmethod
    def backward(ctx, grad_output):
        grads = ctx.inst.apply(grad_output)
        grads = tuple(grads) if isinstance(grads, (tuple, list)) else (grads,)
        if len(grads) != ctx.n:
            raise RuntimeError(f"{ctx.inst.name()}.apply returned {len(grads)} gradients for {ctx.n} inputs")
        return (None, *grads)


_THREAD_GRAPHS = __import__("threading").local()


def with_graph(f):
    """Calls ``f`` with this thread's ``ComputationGraph`` registry (graph.rs:158-163): a graph
    that lives as long as the thread, for code that registers its own leaves and operations."""
    g = getattr(_THREAD_GRAPHS, "graph", None)
    if g is None:
        g = _THREAD_GRAPHS.graph = ComputationGraph()
    return f(g)
