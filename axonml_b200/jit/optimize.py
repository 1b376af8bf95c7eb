"""Graph optimisation passes (crates/axonml-jit/src/optimize.rs:10-190): ConstantFolding,
DeadCodeElimination, ElementwiseFusion, CommonSubexpressionElimination, AlgebraicSimplification,
StrengthReduction; default pipeline = CF, AlgSimp, DCE, CSE.  ``ElementwiseFusion`` marks maximal
groups of same-shape elementwise nodes; the CUDA code generator turns each group into one kernel
(in the reference the pass is a no-op, optimize.rs:178-183)."""
from __future__ import annotations

import enum
import math

from .ir import Graph, Op


class OptimizationPass(enum.Enum):
    ConstantFolding = "constant_folding"
    DeadCodeElimination = "dce"
    ElementwiseFusion = "elementwise_fusion"
    CommonSubexpressionElimination = "cse"
    AlgebraicSimplification = "algebraic_simplification"
    StrengthReduction = "strength_reduction"


_FOLD1 = {"Neg": lambda x: -x, "Abs": abs, "Sqrt": math.sqrt, "Exp": math.exp, "Log": math.log, "Sin": math.sin,
          "Cos": math.cos, "Tanh": math.tanh, "Relu": lambda x: max(x, 0.0),
          "Sigmoid": lambda x: 1 / (1 + math.exp(-x))}
_FOLD2 = {"Add": lambda a, b: a + b, "Sub": lambda a, b: a - b, "Mul": lambda a, b: a * b,
          "Div": lambda a, b: a / b, "Pow": lambda a, b: a ** b, "Max": max, "Min": min}


def _rebuild(g: Graph, keep, replace) -> Graph:
    """New graph with nodes in ``keep`` order; ``replace[id]`` redirects uses."""
    out, remap = Graph(), {}

    def res(i):
        while i in replace:
            i = replace[i]
        return remap[i]
    for n in g.nodes:
        if n.id not in keep or n.id in replace:
            continue
        op = Op(n.op.kind, tuple(res(i) for i in n.op.inputs), n.op.attrs)
        remap[n.id] = out.add_node(op, n.dtype, n.shape)
    return out


class Optimizer:
    def __init__(self, passes=None):
        self.passes = list(passes) if passes is not None else []

    @classmethod
    def new(cls): return cls([])

    @classmethod
    def default_passes(cls):
        return cls([OptimizationPass.ConstantFolding, OptimizationPass.AlgebraicSimplification,
                    OptimizationPass.DeadCodeElimination, OptimizationPass.CommonSubexpressionElimination])

    def add_pass(self, p: OptimizationPass): self.passes.append(p); return self

    def optimize(self, g: Graph) -> Graph:
        for p in self.passes:
            g = {OptimizationPass.ConstantFolding: self.constant_folding,
                 OptimizationPass.DeadCodeElimination: self.dce,
                 OptimizationPass.ElementwiseFusion: self.elementwise_fusion,
                 OptimizationPass.CommonSubexpressionElimination: self.cse,
                 OptimizationPass.AlgebraicSimplification: self.algebraic,
                 OptimizationPass.StrengthReduction: self.strength_reduction}[p](g)
        return g

    # ---- passes
    def constant_folding(self, g: Graph) -> Graph:
        const, out, remap = {}, Graph(), {}
        for n in g.nodes:
            k, ins = n.op.kind, n.op.inputs
            val = None
            if k == "Constant":
                val = n.op.attr("value")
            elif k in _FOLD1 and ins[0] in const:
                try: val = _FOLD1[k](const[ins[0]])
                except (ValueError, OverflowError): val = None
            elif k in _FOLD2 and ins[0] in const and ins[1] in const:
                try: val = _FOLD2[k](const[ins[0]], const[ins[1]])
                except (ValueError, ZeroDivisionError, OverflowError): val = None
            elif k == "AddScalar" and ins[0] in const: val = const[ins[0]] + n.op.attr("scalar")
            elif k == "MulScalar" and ins[0] in const: val = const[ins[0]] * n.op.attr("scalar")
            if val is not None and n.shape == ():
                const[n.id] = float(val)
                remap[n.id] = out.add_node(Op.make("Constant", (), value=float(val)), n.dtype, ())
            else:
                remap[n.id] = out.add_node(Op(k, tuple(remap[i] for i in ins), n.op.attrs), n.dtype, n.shape)
        return out

    def dce(self, g: Graph) -> Graph:
        live, stack = set(), list(g.outputs.values())
        while stack:
            i = stack.pop()
            if i in live:
                continue
            live.add(i)
            stack.extend(g.node(i).op.inputs)
        live |= set(g.inputs.values())
        return _rebuild(g, live, {})

    def cse(self, g: Graph) -> Graph:
        seen, replace = {}, {}
        for n in g.nodes:
            if n.op.kind in ("Input", "Output"):
                continue
            ins = tuple(replace.get(i, i) for i in n.op.inputs)
            key = (n.op.kind, ins, n.op.attrs, n.shape)
            if key in seen:
                replace[n.id] = seen[key]
            else:
                seen[key] = n.id
        return _rebuild(g, {n.id for n in g.nodes}, replace)

    def algebraic(self, g: Graph) -> Graph:
        consts = {n.id: n.op.attr("value") for n in g.nodes if n.op.kind == "Constant"}
        replace = {}
        for n in g.nodes:
            k, ins = n.op.kind, n.op.inputs

            def same_shape(i): return g.node(i).shape == n.shape
            if k in ("Add", "Sub") and consts.get(ins[1]) == 0.0 and same_shape(ins[0]): replace[n.id] = ins[0]
            elif k == "Add" and consts.get(ins[0]) == 0.0 and same_shape(ins[1]): replace[n.id] = ins[1]
            elif k in ("Mul", "Div") and consts.get(ins[1]) == 1.0 and same_shape(ins[0]): replace[n.id] = ins[0]
            elif k == "Mul" and consts.get(ins[0]) == 1.0 and same_shape(ins[1]): replace[n.id] = ins[1]
            elif k == "AddScalar" and n.op.attr("scalar") == 0.0: replace[n.id] = ins[0]
            elif k == "MulScalar" and n.op.attr("scalar") == 1.0: replace[n.id] = ins[0]
            elif k == "Neg" and g.node(ins[0]).op.kind == "Neg": replace[n.id] = g.node(ins[0]).op.inputs[0]
        return _rebuild(g, {n.id for n in g.nodes}, replace)

    def strength_reduction(self, g: Graph) -> Graph:
        consts = {n.id: n.op.attr("value") for n in g.nodes if n.op.kind == "Constant"}
        out, remap = Graph(), {}
        for n in g.nodes:
            k, ins = n.op.kind, tuple(remap[i] for i in n.op.inputs)
            op = Op(k, ins, n.op.attrs)
            if k == "Pow" and consts.get(n.op.inputs[1]) == 2.0: op = Op.make("Mul", (ins[0], ins[0]))
            elif k == "Pow" and consts.get(n.op.inputs[1]) == 0.5: op = Op.make("Sqrt", (ins[0],))
            elif k == "Div" and n.op.inputs[1] in consts and consts[n.op.inputs[1]] not in (0.0, None):
                op = Op.make("MulScalar", (ins[0],), scalar=1.0 / consts[n.op.inputs[1]])
            elif k == "Mul" and consts.get(n.op.inputs[1]) == 2.0: op = Op.make("Add", (ins[0], ins[0]))
            remap[n.id] = out.add_node(op, n.dtype, n.shape)
        return out

    def elementwise_fusion(self, g: Graph) -> Graph:
        """Annotates nodes with a ``fusion_group`` attribute (consumed by the code generator)."""
        group_of, next_group = {}, 0
        out = Graph()
        for n in g.nodes:
            attrs = n.op.attrs
            if n.op.is_elementwise() and n.op.kind != "Constant" and n.shape != ():
                gid = None
                for i in n.op.inputs:
                    if i in group_of and g.node(i).shape == n.shape:
                        gid = group_of[i]
                        break
                if gid is None:
                    gid, next_group = next_group, next_group + 1
                group_of[n.id] = gid
                attrs = tuple(sorted(dict(attrs, fusion_group=gid).items()))
            out.add_node(Op(n.op.kind, n.op.inputs, attrs), n.dtype, n.shape)
        return out
