"""JIT: IR, tracer, passes, cache, executors (crates/axonml-jit)."""
from .cache import CacheStats, FunctionCache
from .codegen import CompiledFunction, JitCompiler, generate_cuda, interpret
from .compile import (Backend, CompileConfig, CompiledModel, CompileStats, LazyCompiled, Mode, compile_fn,
                      compile_fn_with_config, compile_graph, compile_graph_with_config)
from . import error
from .error import JitError
from .ir import DataType, Graph, Node, NodeId, Op, Shape
from .optimize import OptimizationPass, Optimizer
from .trace import TracedValue, Tracer, trace
