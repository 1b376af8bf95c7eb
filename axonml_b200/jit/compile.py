"""torch.compile-like front end (crates/axonml-jit/src/compile.rs:39-502): ``Mode``, ``Backend``,
``CompileConfig`` builder, ``CompiledModel``, ``compile_graph`` / ``compile_fn`` and
``LazyCompiled``."""
from __future__ import annotations

import dataclasses
import enum

from .codegen import CompiledFunction, JitCompiler
from .ir import Graph
from .optimize import OptimizationPass, Optimizer
from .trace import trace


class Mode(enum.Enum):
    Default = "default"
    ReduceOverhead = "reduce-overhead"
    MaxAutotune = "max-autotune"


class Backend(enum.Enum):
    Default = "default"
    Interpreter = "interpreter"
    Cuda = "cuda"


@dataclasses.dataclass
class CompileStats:
    original_nodes: int
    optimized_nodes: int
    passes: int
    generated_kernel: bool = False

    def optimization_ratio(self) -> float:
        return 1.0 - self.optimized_nodes / self.original_nodes if self.original_nodes else 0.0


class CompileConfig:
    def __init__(self):
        self._mode, self._backend = Mode.Default, Backend.Default
        self._fullgraph, self._dynamic, self._disable = False, False, False
        self._passes: list = []

    @classmethod
    def new(cls): return cls()
    def mode(self, m: Mode): self._mode = m; return self
    def backend(self, b: Backend): self._backend = b; return self
    def fullgraph(self, f: bool): self._fullgraph = f; return self
    def dynamic(self, d: bool): self._dynamic = d; return self
    def disable(self, d: bool): self._disable = d; return self
    def add_pass(self, p: OptimizationPass): self._passes.append(p); return self

    def optimizer(self) -> Optimizer:
        if self._disable:
            return Optimizer.new()
        opt = Optimizer.default_passes()
        if self._mode is not Mode.Default:
            opt.add_pass(OptimizationPass.StrengthReduction).add_pass(OptimizationPass.ElementwiseFusion)
        for p in self._passes:
            opt.add_pass(p)
        return opt


class CompiledModel:
    def __init__(self, graph: Graph, config: CompileConfig):
        self._graph, self._config = graph, config
        self._fn: CompiledFunction = JitCompiler.with_optimizer(config.optimizer()).compile(graph)

    @classmethod
    def from_graph(cls, graph: Graph, config: CompileConfig | None = None): return cls(graph, config or CompileConfig())
    def input_names(self): return self._graph.input_names()
    def output_names(self): return self._graph.output_names()
    def graph(self) -> Graph: return self._graph
    def optimized_graph(self) -> Graph: return self._fn.graph()
    def is_compiled(self) -> bool: return True
    def stats(self) -> CompileStats:
        return CompileStats(len(self._graph), len(self._fn.graph()), len(self._config.optimizer().passes),
                            self._fn.uses_generated_kernel())
    def run(self, inputs: dict) -> dict: return self._fn.run(dict(inputs))
    def run_tensors(self, inputs: dict) -> dict: return self._fn.run_tensors(inputs)


def compile_graph(graph: Graph) -> CompiledModel: return CompiledModel(graph, CompileConfig())
def compile_graph_with_config(graph: Graph, config: CompileConfig) -> CompiledModel: return CompiledModel(graph, config)
def compile_fn(fn) -> CompiledModel: return compile_graph(trace(fn))
def compile_fn_with_config(fn, config: CompileConfig) -> CompiledModel: return CompiledModel(trace(fn), config)


class LazyCompiled:
    def __init__(self, fn, config: CompileConfig | None = None):
        self._fn, self._config, self._model = fn, config or CompileConfig(), None

    @classmethod
    def new(cls, fn): return cls(fn)
    @classmethod
    def with_config(cls, fn, config): return cls(fn, config)

    def run(self, inputs: dict) -> dict:
        if self._model is None:
            self._model = compile_fn_with_config(self._fn, self._config)
        return self._model.run(inputs)
