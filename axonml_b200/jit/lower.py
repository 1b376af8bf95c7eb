"""Lowering of a whole IR graph to generated CUDA kernels (compiled with NVRTC for the GPU at hand).

Where ``codegen.generate_cuda`` covers the one-kernel case (a same-shape elementwise expression),
this module lowers every graph of the IR (crates/axonml-jit/src/ir.rs:139-262: elementwise ops with
implicit broadcasting, ``Broadcast`` / ``Reshape`` / ``Squeeze`` / ``Unsqueeze`` / ``Transpose``,
``Where``, ``Cast``, full and per-axis reductions, ``MatMul``) to a short sequence of launches:

* some nodes are *materialised* in device buffers: inputs, reductions, matrix products and their
  operands, output values, and values with several users (so that nothing is recomputed);
* every other node is fused into the kernel of the materialised node that consumes it: the generator
  walks the expression down to materialised leaves and emits the index arithmetic of broadcasts,
  transposes and reshapes as it goes (a leaf is read at the offset its own shape gives it);
* a reduction becomes one kernel with a warp (or a 256-thread block for long rows) per output
  element that evaluates the fused producer expression while it reduces; a reduction to a single
  value over a large tensor is split over blocks that combine with one atomic add each;
* ``MatMul`` runs on the library's fp32 GEMM kernel.

Values are fp32 in registers and buffers (comparison results are 0 / 1); outputs are converted to
their declared dtype at the end.  The reference executes the same graphs with a per-node
interpreter (codegen.rs:77-368); ``codegen.interpret`` is this package's counterpart and the
fallback on machines without a GPU.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .error import UnsupportedOp
from .ir import Graph

_UN = {"Neg": "(-{0})", "Abs": "fabsf({0})", "Sqrt": "sqrtf({0})", "Exp": "__expf({0})", "Log": "__logf({0})",
       "Sin": "__sinf({0})", "Cos": "__cosf({0})", "Tanh": "tanhf({0})", "Relu": "fmaxf({0}, 0.f)",
       "Sigmoid": "(1.f / (1.f + __expf(-{0})))",
       "Gelu": "(0.5f * {0} * (1.f + tanhf(0.7978845608f * ({0} + 0.044715f * {0} * {0} * {0}))))",
       "Silu": "({0} / (1.f + __expf(-{0})))", "Contiguous": "{0}"}
_BIN = {"Add": "({0} + {1})", "Sub": "({0} - {1})", "Mul": "({0} * {1})", "Div": "({0} / {1})",
        "Pow": "powf({0}, {1})", "Max": "fmaxf({0}, {1})", "Min": "fminf({0}, {1})",
        "Gt": "(({0} > {1}) ? 1.f : 0.f)", "Lt": "(({0} < {1}) ? 1.f : 0.f)", "Eq": "(({0} == {1}) ? 1.f : 0.f)"}
_VIEW = ("Reshape", "Squeeze", "Unsqueeze", "Contiguous")
_REDUCE = ("Sum", "Mean", "SumAxis", "MeanAxis", "MaxAxis")
_TORCH_DT = {"f32": torch.float32, "f64": torch.float64, "i32": torch.int32, "i64": torch.int64, "bool": torch.bool}


def _numel(shape) -> int:
    return int(math.prod(shape)) if len(shape) else 1


def _lit(x: float) -> str:
    if math.isinf(x):       # NVRTC compiles without <cmath>: spell the bit patterns
        return "__int_as_float(0x7f800000)" if x > 0 else "__int_as_float(0xff800000)"
    if math.isnan(x):
        return "__int_as_float(0x7fffffff)"
    return f"{float(x)!r}f"


class _KernelBuilder:
    """Statements of one kernel body; expressions are memoised per (node, index variable)."""

    def __init__(self, graph: Graph, materialised: set):
        self.g, self.mat = graph, materialised
        self.stmts: list[str] = []
        self.memo: dict = {}
        self.leaves: list[int] = []      # materialised nodes this kernel reads, in parameter order
        self._tmp = 0

    def _new(self, prefix: str) -> str:
        self._tmp += 1
        return f"{prefix}{self._tmp}"

    def _index_into(self, idx: str, from_shape, to_shape, perm=None) -> str:
        """Index variable for reading a tensor of ``to_shape`` at the element that position ``idx`` of
        ``from_shape`` maps to: right-aligned broadcasting (size-1 and missing dims repeat), after an
        optional swap of two dims of the multi-index (``perm`` = (d0, d1), for Transpose)."""
        if tuple(from_shape) == tuple(to_shape) and perm is None:
            return idx
        if _numel(to_shape) == 1:
            return "0"
        name = self._new("i")
        coords, rem = [], idx
        lines = []
        r = self._new("r")
        lines.append(f"long {r} = {idx};")
        for d in reversed(range(len(from_shape))):
            c = self._new("c")
            lines.append(f"const long {c} = {r} % {from_shape[d]}L; {r} /= {from_shape[d]}L;")
            coords.append(c)
        coords.reverse()
        if perm is not None:
            coords[perm[0]], coords[perm[1]] = coords[perm[1]], coords[perm[0]]
        # strides of the target, right-aligned against the (possibly permuted) source coordinates
        terms, stride = [], 1
        off = len(coords) - len(to_shape)
        for d in reversed(range(len(to_shape))):
            if to_shape[d] != 1 and off + d >= 0:
                terms.append(f"{coords[off + d]} * {stride}L")
            stride *= to_shape[d]
        lines.append(f"const long {name} = {' + '.join(terms) if terms else '0'};")
        self.stmts.extend(lines)
        return name

    def value(self, nid: int, idx: str, root: bool = False) -> str:
        """C expression of node ``nid`` at linear position ``idx`` of its own shape."""
        key = (nid, idx)
        if key in self.memo:
            return self.memo[key]
        n = self.g.node(nid)
        k = n.op.kind
        if nid in self.mat and not root:
            if nid not in self.leaves:
                self.leaves.append(nid)
            e = f"b{nid}[{idx}]" if _numel(n.shape) > 1 else f"b{nid}[0]"
            self.memo[key] = e
            return e
        ins = n.op.inputs

        def arg(j):
            src = self.g.node(ins[j])
            return self.value(ins[j], self._index_into(idx, n.shape, src.shape))
        if k == "Constant":
            e = _lit(n.op.attr("value"))
        elif k in _UN:
            e = _UN[k].format(arg(0))
        elif k in _BIN:
            e = _BIN[k].format(arg(0), arg(1))
        elif k == "AddScalar":
            e = f"({arg(0)} + {_lit(n.op.attr('scalar'))})"
        elif k == "MulScalar":
            e = f"({arg(0)} * {_lit(n.op.attr('scalar'))})"
        elif k == "Where":
            e = f"(({arg(0)} != 0.f) ? {arg(1)} : {arg(2)})"
        elif k == "Cast":
            dt = n.op.attr("dtype")
            e = f"truncf({arg(0)})" if dt in ("i32", "i64") else (f"(({arg(0)} != 0.f) ? 1.f : 0.f)" if dt == "bool" else arg(0))
        elif k in ("Reshape", "Squeeze", "Unsqueeze"):
            e = self.value(ins[0], idx)                       # the linear position does not change
        elif k == "Broadcast":
            e = self.value(ins[0], self._index_into(idx, n.shape, self.g.node(ins[0]).shape))
        elif k == "Transpose":
            src = self.g.node(ins[0])
            e = self.value(ins[0], self._index_into(idx, n.shape, src.shape, (n.op.attr("dim0") % len(n.shape), n.op.attr("dim1") % len(n.shape))))
        elif k == "Output":
            e = self.value(ins[0], idx)
        else:
            raise UnsupportedOp(k)
        v = self._new("v")
        self.stmts.append(f"const float {v} = {e};")
        self.memo[key] = v
        return v


class Plan:
    """Generated module plus the launches that evaluate a graph."""

    def __init__(self, graph: Graph):
        self.graph = graph
        self.steps: list[dict] = []
        self.kernels: dict = {}
        self.source = ""
        self._lower()

    # ------------------------------------------------------------------ analysis
    def _materialised(self) -> set:
        g = self.graph
        users = g.users()
        mat = set()
        for n in g.nodes:
            k = n.op.kind
            if k == "Input" or k in _REDUCE or k == "MatMul":
                mat.add(n.id)
            if k == "MatMul":
                mat.update(n.op.inputs)
            if k == "Output":
                mat.add(n.op.inputs[0])
        for n in g.nodes:
            if n.id in mat or n.op.kind in ("Constant", "Output", "Input"):
                continue
            real = [u for u in users[n.id]]
            if len(real) > 1 and n.op.kind not in _VIEW + ("Broadcast",):
                mat.add(n.id)
        return mat

    # ------------------------------------------------------------------ code generation
    def _lower(self) -> None:
        g = self.graph
        mat = self._materialised()
        src = []
        for n in g.nodes:
            k = n.op.kind
            if n.id not in mat or k == "Input":
                continue
            if k == "MatMul":
                self.steps.append({"kind": "matmul", "out": n.id, "a": n.op.inputs[0], "b": n.op.inputs[1]})
                continue
            kb = _KernelBuilder(g, mat)
            name = f"axonml_k{n.id}"
            if k in _REDUCE:
                x = g.node(n.op.inputs[0])
                if k in ("Sum", "Mean"):
                    outer, red, inner = 1, _numel(x.shape), 1
                else:
                    a = n.op.attr("axis")
                    outer, red, inner = _numel(x.shape[:a]), x.shape[a], _numel(x.shape[a + 1:])
                is_max = k == "MaxAxis"
                split = 1
                if outer * inner == 1 and not is_max and red >= (1 << 16):
                    split = min(1024, (red + 8191) // 8192)
                threads = 256 if red // split >= 2048 else 32
                val = kb.value(x.id, "xl")
                body = "\n      ".join(kb.stmts)
                params = ", ".join([f"const float* __restrict__ b{l}" for l in kb.leaves] + ["float* __restrict__ out"])
                comb = "fmaxf(acc, {0})" if is_max else "(acc + {0})"
                init = "__int_as_float(0xff800000)" if is_max else "0.f"
                scale = f" * {1.0 / red!r}f" if k in ("Mean", "MeanAxis") else ""
                src.append(f"""
extern "C" __global__ void __launch_bounds__({threads}) {name}({params}) {{
  // one output element per group of {threads} threads; `part` splits a long reduction over blocks
  const long o = (long)blockIdx.x / {split};
  const int part = (int)(blockIdx.x % {split});
  if (o >= {outer * inner}L) return;
  const long oi = o / {inner}L, ii = o % {inner}L;
  const long per = ({red}L + {split} - 1) / {split};
  const long j0 = part * per, j1 = (j0 + per < {red}L) ? j0 + per : {red}L;
  float acc = {init};
  for (long j = j0 + threadIdx.x; j < j1; j += {threads}) {{
      const long xl = (oi * {red}L + j) * {inner}L + ii;
      {body}
      acc = {comb.format(val)};
  }}
  for (int s = 16; s > 0; s >>= 1) {{ const float t = __shfl_xor_sync(0xffffffffu, acc, s); acc = {comb.format('t')}; }}
  __shared__ float red_smem[8];
  if ({threads} > 32) {{
    if ((threadIdx.x & 31) == 0) red_smem[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {{
      acc = threadIdx.x < {threads // 32} ? red_smem[threadIdx.x] : {init};
      for (int s = 16; s > 0; s >>= 1) {{ const float t = __shfl_xor_sync(0xffffffffu, acc, s); acc = {comb.format('t')}; }}
    }}
  }}
  if (threadIdx.x == 0) {{
    if ({split} > 1) atomicAdd(out + o, acc{scale}); else out[o] = acc{scale};
  }}
}}
""")
                self.steps.append({"kind": "kernel", "name": name, "out": n.id, "leaves": list(kb.leaves),
                                   "grid": outer * inner * split, "block": threads, "zero": split > 1, "n": None})
            else:
                val = kb.value(n.id, "lin", root=True)
                body = "\n    ".join(kb.stmts)
                params = ", ".join([f"const float* __restrict__ b{l}" for l in kb.leaves] + ["float* __restrict__ out", "long total"])
                src.append(f"""
extern "C" __global__ void __launch_bounds__(256) {name}({params}) {{
  for (long lin = (long)blockIdx.x * blockDim.x + threadIdx.x; lin < total; lin += (long)gridDim.x * blockDim.x) {{
    {body}
    out[lin] = {val};
  }}
}}
""")
                total = _numel(n.shape)
                self.steps.append({"kind": "kernel", "name": name, "out": n.id, "leaves": list(kb.leaves),
                                   "grid": max(1, min((total + 255) // 256, 148 * 16)), "block": 256, "zero": False, "n": total})
        self.source = "".join(src)

    # ------------------------------------------------------------------ execution
    def compile(self) -> None:
        from . import nvrtc
        if not self.source:
            return
        mod = nvrtc.Module(self.source)
        for st in self.steps:
            if st["kind"] == "kernel":
                self.kernels[st["name"]] = mod.function(st["name"])

    def run(self, inputs: dict) -> dict:
        g = self.graph
        dev = next(iter(inputs.values())).device
        buf: dict = {}
        for name, nid in g.inputs.items():
            t = inputs[name].to(device=dev, dtype=torch.float32).contiguous()
            want = g.node(nid).shape
            if tuple(t.shape) != tuple(want) and t.numel() == _numel(want):
                t = t.reshape(want)
            buf[nid] = t
        for st in self.steps:
            n = g.node(st["out"])
            if st["kind"] == "matmul":
                from ..ops.gemm import sgemm_f32
                a, b = buf[st["a"]], buf[st["b"]]
                if a.dim() in (2, 3) and b.dim() in (2, 3) and (a.dim() == b.dim() or b.dim() == 2):
                    buf[n.id] = sgemm_f32(a, b).reshape(n.shape)
                else:
                    buf[n.id] = torch.matmul(a, b).reshape(n.shape).contiguous()
                continue
            out = (torch.zeros if st["zero"] else torch.empty)(n.shape if len(n.shape) else (1,), dtype=torch.float32, device=dev)
            args = [buf[l].data_ptr() for l in st["leaves"]] + [out.data_ptr()]
            types = [ctypes.c_void_p] * len(args)
            if st["n"] is not None:
                args.append(st["n"])
                types.append(ctypes.c_long)
            self.kernels[st["name"]].launch(st["grid"], st["block"], args, types)
            buf[n.id] = out.reshape(n.shape) if len(n.shape) else out.reshape(())
        outs = {}
        for name, nid in g.outputs.items():
            node = g.node(nid)
            t = buf[node.op.inputs[0]]
            dt = _TORCH_DT[node.dtype.value]
            outs[name] = t if dt == torch.float32 else t.to(dt)
        return outs


def lowerable(graph: Graph) -> bool:
    known = set(_UN) | set(_BIN) | set(_REDUCE) | {"Input", "Output", "Constant", "AddScalar", "MulScalar", "Where",
                                                    "Cast", "Reshape", "Squeeze", "Unsqueeze", "Broadcast",
                                                    "Transpose", "MatMul"}
    return bool(graph.outputs) and all(n.op.kind in known for n in graph.nodes)
