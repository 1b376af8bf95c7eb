"""Executors for compiled graphs (crates/axonml-jit/src/codegen.rs:14-741).

``JitCompiler.compile(graph)`` optimises the graph, looks it up in the ``FunctionCache`` and
returns a ``CompiledFunction``.  Executors: an interpreter over torch ops (any device, every op);
on CUDA, generated kernels compiled with NVRTC for sm_100a: one kernel when the graph is a single
same-shape elementwise expression, else the multi-kernel plan of ``lower.py`` (broadcasting, shape
ops, ``Where`` / ``Cast``, reductions fused with their producer expressions, ``MatMul`` on the
library GEMM).  The reference's native path, Cranelift, is unreachable there (``use_native:
false``, codegen.rs:503)."""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from .cache import FunctionCache
from .error import InputNotFound, OutputNotFound, ShapeMismatch, UnsupportedOp
from .ir import Graph
from .optimize import Optimizer

_TORCH_DT = {"f32": torch.float32, "f64": torch.float64, "i32": torch.int32, "i64": torch.int64, "bool": torch.bool}


def interpret(graph: Graph, inputs: dict) -> dict:
    v: dict = {}
    outs = {}
    for n in graph.nodes:
        k, a = n.op.kind, [v[i] for i in n.op.inputs]
        at = n.op.attr
        if k == "Input":
            if at("name") not in inputs:
                raise InputNotFound(at("name"))
            r = inputs[at("name")]
        elif k == "Output":
            r = a[0]
            outs[at("name")] = r
        elif k == "Constant": r = torch.tensor(at("value"), dtype=torch.float32, device=_dev(inputs))
        elif k == "Add": r = a[0] + a[1]
        elif k == "Sub": r = a[0] - a[1]
        elif k == "Mul": r = a[0] * a[1]
        elif k == "Div": r = a[0] / a[1]
        elif k == "Pow": r = a[0] ** a[1]
        elif k == "Max": r = torch.maximum(a[0], a[1])
        elif k == "Min": r = torch.minimum(a[0], a[1])
        elif k == "Neg": r = -a[0]
        elif k == "Abs": r = a[0].abs()
        elif k == "Sqrt": r = a[0].sqrt()
        elif k == "Exp": r = a[0].exp()
        elif k == "Log": r = a[0].log()
        elif k == "Sin": r = a[0].sin()
        elif k == "Cos": r = a[0].cos()
        elif k == "Tanh": r = a[0].tanh()
        elif k == "Relu": r = a[0].relu()
        elif k == "Sigmoid": r = a[0].sigmoid()
        elif k == "Gelu": r = F.gelu(a[0], approximate="tanh")
        elif k == "Silu": r = F.silu(a[0])
        elif k == "AddScalar": r = a[0] + at("scalar")
        elif k == "MulScalar": r = a[0] * at("scalar")
        elif k == "Sum": r = a[0].sum()
        elif k == "Mean": r = a[0].mean()
        elif k == "SumAxis": r = a[0].sum(at("axis"), at("keepdim"))
        elif k == "MeanAxis": r = a[0].mean(at("axis"), at("keepdim"))
        elif k == "MaxAxis": r = a[0].max(at("axis"), at("keepdim")).values
        elif k == "Reshape": r = a[0].reshape(n.shape)
        elif k == "Transpose": r = a[0].transpose(at("dim0"), at("dim1"))
        elif k == "Squeeze": r = a[0].squeeze(at("dim"))
        elif k == "Unsqueeze": r = a[0].unsqueeze(at("dim"))
        elif k == "Broadcast": r = a[0].expand(n.shape)
        elif k == "MatMul": r = a[0] @ a[1]
        elif k == "Gt": r = a[0] > a[1]
        elif k == "Lt": r = a[0] < a[1]
        elif k == "Eq": r = a[0] == a[1]
        elif k == "Where": r = torch.where(a[0].bool(), a[1], a[2])
        elif k == "Cast": r = a[0].to(_TORCH_DT[at("dtype")])
        elif k == "Contiguous": r = a[0].contiguous()
        else: raise UnsupportedOp(k)
        v[n.id] = r
    return outs


def _dev(inputs):
    for t in inputs.values():
        return t.device
    return "cpu"


_EXPR = {"Add": "({0} + {1})", "Sub": "({0} - {1})", "Mul": "({0} * {1})", "Div": "({0} / {1})",
         "Pow": "powf({0}, {1})", "Max": "fmaxf({0}, {1})", "Min": "fminf({0}, {1})", "Neg": "(-{0})",
         "Abs": "fabsf({0})", "Sqrt": "sqrtf({0})", "Exp": "__expf({0})", "Log": "__logf({0})",
         "Sin": "__sinf({0})", "Cos": "__cosf({0})", "Tanh": "tanhf({0})", "Relu": "fmaxf({0}, 0.f)",
         "Sigmoid": "(1.f / (1.f + __expf(-{0})))",
         "Gelu": "(0.5f * {0} * (1.f + tanhf(0.7978845608f * ({0} + 0.044715f * {0} * {0} * {0}))))",
         "Silu": "({0} / (1.f + __expf(-{0})))", "Gt": "(({0} > {1}) ? 1.f : 0.f)",
         "Lt": "(({0} < {1}) ? 1.f : 0.f)", "Eq": "(({0} == {1}) ? 1.f : 0.f)",
         "Where": "(({0} != 0.f) ? {1} : {2})", "Contiguous": "{0}", "Cast": "{0}"}


def generate_cuda(graph: Graph):
    """CUDA C for a graph that is a single same-shape fp32 elementwise expression, or None."""
    shape = None
    for n in graph.nodes:
        if n.op.kind in ("Input", "Output") or n.op.is_elementwise():
            if n.shape != ():
                if shape is None:
                    shape = n.shape
                elif n.shape != shape:
                    return None
            if n.dtype.value not in ("f32", "bool"):
                return None
        else:
            return None
    if shape is None or not graph.outputs:
        return None
    ins = list(graph.inputs.items())
    outs = list(graph.outputs.items())
    params = [f"const float* __restrict__ in{i}" for i in range(len(ins))] + [f"float* __restrict__ out{i}" for i in range(len(outs))]
    body = []
    name_of = {}
    for n in graph.nodes:
        k = n.op.kind
        a = [name_of[i] for i in n.op.inputs]
        if k == "Input":
            idx = [i for i, (_, nid) in enumerate(ins) if nid == n.id][0]
            expr = f"in{idx}[0]" if n.shape == () else f"in{idx}[i]"
        elif k == "Constant": expr = f"{float(n.op.attr('value'))!r}f".replace("-inff", "__int_as_float(0xff800000)").replace("inff", "__int_as_float(0x7f800000)").replace("nanf", "__int_as_float(0x7fffffff)")
        elif k == "AddScalar": expr = f"({a[0]} + {float(n.op.attr('scalar'))!r}f)"
        elif k == "MulScalar": expr = f"({a[0]} * {float(n.op.attr('scalar'))!r}f)"
        elif k == "Output":
            idx = [i for i, (_, nid) in enumerate(outs) if nid == n.id][0]
            body.append(f"    out{idx}[i] = {a[0]};")
            continue
        else:
            expr = _EXPR[k].format(*a)
        name_of[n.id] = f"v{n.id}"
        body.append(f"    const float v{n.id} = {expr};")
    src = ("extern \"C\" __global__ void axonml_fused(" + ", ".join(params) + ", long n) {\n"
           "  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {\n"
           + "\n".join(body) + "\n  }\n}\n")
    return src, [k for k, _ in ins], [k for k, _ in outs], shape


class CompiledFunction:
    def __init__(self, graph: Graph, original: Graph | None = None):
        self._graph, self._original = graph, original or graph
        self._kernel, self._cuda = None, None
        self._plan = None
        self._tried_cuda = False

    @classmethod
    def placeholder(cls): return cls(Graph())

    def graph(self) -> Graph: return self._graph
    def uses_generated_kernel(self) -> bool: return self._kernel is not None or self._plan is not None

    def generated_source(self) -> str | None:
        """CUDA C of the generated kernels (after the first run on a GPU), for inspection."""
        if self._kernel is not None:
            return self._cuda[0]
        return self._plan.source if self._plan is not None else None

    def _try_cuda(self) -> None:
        self._tried_cuda = True
        from . import nvrtc
        if not nvrtc.available():
            return
        gen = generate_cuda(self._graph)
        if gen is not None:
            self._cuda = gen
            self._kernel = nvrtc.Kernel(gen[0], "axonml_fused")
            return
        from . import lower
        if lower.lowerable(self._graph):
            plan = lower.Plan(self._graph)
            plan.compile()
            self._plan = plan

    def run_tensors(self, inputs: dict) -> dict:
        """Tensor-level entry: ``{name: tensor}`` -> ``{name: tensor}``."""
        first = next(iter(inputs.values())) if inputs else None
        if first is not None and first.is_cuda and all(t.dtype == torch.float32 for t in inputs.values()):
            if not self._tried_cuda:
                self._try_cuda()
            if self._kernel is not None:
                _, in_names, out_names, shape = self._cuda
                n = 1
                for s in shape:
                    n *= s
                ins = [inputs[k].contiguous() for k in in_names]
                outs = [torch.empty(shape, dtype=torch.float32, device=first.device) for _ in out_names]
                args = [t.data_ptr() for t in ins] + [t.data_ptr() for t in outs] + [n]
                types = [ctypes.c_void_p] * (len(ins) + len(outs)) + [ctypes.c_long]
                grid = max(1, min((n + 255) // 256, 148 * 16))
                self._kernel.launch(grid, 256, args, types)
                return dict(zip(out_names, outs))
        if first is not None and first.is_cuda:
            if not self._tried_cuda:
                self._try_cuda()
            if self._plan is not None:
                return self._plan.run(inputs)
        return interpret(self._graph, inputs)

    def run(self, inputs):
        """Reference-shaped entry: ``[(name, values)]`` -> flat list of the (first) output."""
        g = self._graph
        tin = {}
        for name, vals in (inputs.items() if isinstance(inputs, dict) else inputs):
            if name not in g.inputs:
                raise InputNotFound(name)
            t = torch.as_tensor(vals, dtype=torch.float32)
            want = g.node(g.inputs[name]).shape
            if t.dim() <= 1:
                n = 1
                for d in want:
                    n *= d
                if t.numel() != n:
                    raise ShapeMismatch(want, t.shape)
                t = t.reshape(want)
            tin[name] = t
        missing = [k for k in g.inputs if k not in tin]
        if missing:
            raise InputNotFound(missing[0])
        outs = self.run_tensors(tin)
        if isinstance(inputs, dict):
            return {k: v.reshape(-1).tolist() for k, v in outs.items()}
        if not outs:
            raise OutputNotFound("the graph declares no output")
        return next(iter(outs.values())).reshape(-1).tolist()


class JitCompiler:
    def __init__(self, optimizer: Optimizer | None = None, cache_size: int = 1000):
        self.optimizer = optimizer or Optimizer.default_passes()
        self.cache = FunctionCache(cache_size)
        self.use_native = True

    @classmethod
    def new(cls): return cls()
    @classmethod
    def with_optimizer(cls, optimizer): return cls(optimizer)

    def compile(self, graph: Graph) -> CompiledFunction:
        graph.validate()
        key = FunctionCache.hash_graph(graph)
        f = self.cache.get(key)
        if f is None:
            f = CompiledFunction(self.optimizer.optimize(graph), graph)
            self.cache.insert(key, f)
        return f

    def cache_stats(self): return self.cache.stats()
    def clear_cache(self) -> None: self.cache.clear()
