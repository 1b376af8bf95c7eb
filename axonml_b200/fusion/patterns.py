"""Fusion pattern detection over a flat op list (crates/axonml-fusion/src/patterns.rs:57-230) and
the ``FusionOptimizer`` / ``FusionConfig`` statistics front end (optimizer.rs:17-215).  The
per-pattern speed-ups are the reference's fixed estimates (patterns.rs:57-73); ``fold_conv_bn``
additionally performs the Conv+BN folding for inference."""
from __future__ import annotations

import dataclasses
import enum

import torch


class OpType(enum.Enum):
    MatMul = "matmul"
    Conv = "conv"
    Add = "add"
    Mul = "mul"
    Relu = "relu"
    Gelu = "gelu"
    Sigmoid = "sigmoid"
    Tanh = "tanh"
    BatchNorm = "batchnorm"
    LayerNorm = "layernorm"
    Softmax = "softmax"
    Exp = "exp"
    Log = "log"
    Sqrt = "sqrt"
    Other = "other"

    def is_elementwise(self) -> bool:
        return self in (OpType.Add, OpType.Mul, OpType.Relu, OpType.Gelu, OpType.Sigmoid, OpType.Tanh,
                        OpType.Exp, OpType.Log, OpType.Sqrt)


class FusionPattern(enum.Enum):
    MatMulBias = "matmul_bias"
    MatMulBiasRelu = "matmul_bias_relu"
    MatMulBiasGelu = "matmul_bias_gelu"
    ConvBatchNorm = "conv_bn"
    ConvBatchNormRelu = "conv_bn_relu"
    AddRelu = "add_relu"
    MulAdd = "mul_add"
    ElementwiseChain = "elementwise_chain"
    Softmax = "softmax"
    LayerNorm = "layernorm"
    GeluApprox = "gelu_approx"

    def estimated_speedup(self) -> float:
        return {FusionPattern.ElementwiseChain: 2.0, FusionPattern.AddRelu: 1.8, FusionPattern.MulAdd: 1.5,
                FusionPattern.ConvBatchNormRelu: 1.4, FusionPattern.MatMulBiasRelu: 1.3,
                FusionPattern.MatMulBiasGelu: 1.3, FusionPattern.ConvBatchNorm: 1.3,
                FusionPattern.MatMulBias: 1.2, FusionPattern.Softmax: 1.2, FusionPattern.LayerNorm: 1.2,
                FusionPattern.GeluApprox: 1.2}[self]

    def is_memory_bound(self) -> bool:
        """Patterns whose cost is memory traffic, where fusing saves whole passes over the data."""
        return self in (FusionPattern.ElementwiseChain, FusionPattern.AddRelu, FusionPattern.MulAdd)

    def num_ops(self) -> int:
        return {FusionPattern.MatMulBias: 2, FusionPattern.MatMulBiasRelu: 3, FusionPattern.MatMulBiasGelu: 3,
                FusionPattern.ConvBatchNorm: 2, FusionPattern.ConvBatchNormRelu: 3, FusionPattern.AddRelu: 2,
                FusionPattern.MulAdd: 2}.get(self, 1)


def detect_patterns(ops) -> list:
    """Greedy left-to-right scan; returns ``(pattern, start, length)`` tuples."""
    ops = list(ops)
    out, i = [], 0
    O = OpType
    while i < len(ops):
        nxt = ops[i + 1] if i + 1 < len(ops) else None
        nn2 = ops[i + 2] if i + 2 < len(ops) else None
        if ops[i] is O.MatMul and nxt is O.Add:
            if nn2 is O.Relu: out.append((FusionPattern.MatMulBiasRelu, i, 3)); i += 3
            elif nn2 is O.Gelu: out.append((FusionPattern.MatMulBiasGelu, i, 3)); i += 3
            else: out.append((FusionPattern.MatMulBias, i, 2)); i += 2
        elif ops[i] is O.Conv and nxt is O.BatchNorm:
            if nn2 is O.Relu: out.append((FusionPattern.ConvBatchNormRelu, i, 3)); i += 3
            else: out.append((FusionPattern.ConvBatchNorm, i, 2)); i += 2
        elif ops[i] is O.Add and nxt is O.Relu: out.append((FusionPattern.AddRelu, i, 2)); i += 2
        elif ops[i] is O.Mul and nxt is O.Add: out.append((FusionPattern.MulAdd, i, 2)); i += 2
        elif ops[i].is_elementwise():
            j = i
            while j < len(ops) and ops[j].is_elementwise():
                j += 1
            if j - i >= 2: out.append((FusionPattern.ElementwiseChain, i, j - i))
            i = j if j > i else i + 1
        elif ops[i] is O.Softmax: out.append((FusionPattern.Softmax, i, 1)); i += 1
        elif ops[i] is O.LayerNorm: out.append((FusionPattern.LayerNorm, i, 1)); i += 1
        else: i += 1
    return out


@dataclasses.dataclass
class FusionConfig:
    fuse_elementwise: bool = True
    fuse_linear: bool = True
    fuse_conv: bool = True
    min_chain_length: int = 2
    aggressive: bool = False

    @classmethod
    def new(cls): return cls()
    @classmethod
    def all_enabled(cls):
        """Every fusion on, chains from two operations, aggressive mode."""
        return cls(True, True, True, 2, True)
    @classmethod
    def conservative(cls): return cls(min_chain_length=3)
    @classmethod
    def aggressive_mode(cls): return cls(aggressive=True)


@dataclasses.dataclass
class FusionStats:
    total_ops: int = 0
    fused_ops: int = 0
    patterns_found: int = 0
    estimated_speedup: float = 1.0

    def fusion_ratio(self) -> float: return self.fused_ops / self.total_ops if self.total_ops else 0.0


@dataclasses.dataclass
class OptimizationStats:
    """Running totals of an optimizer (crates/axonml-fusion/src/optimizer.rs:81-105): each fusion
    removes ``pattern.num_ops() - 1`` operations and multiplies the estimated speedup."""
    fusions_applied: int = 0
    ops_eliminated: int = 0
    estimated_speedup: float = 1.0
    patterns: list = dataclasses.field(default_factory=list)          # [pattern, count] pairs, first seen first

    def add_fusion(self, pattern: FusionPattern, length: int | None = None) -> None:
        self.fusions_applied += 1
        self.ops_eliminated += (length if length is not None else pattern.num_ops()) - 1
        self.estimated_speedup *= pattern.estimated_speedup()
        for entry in self.patterns:
            if entry[0] is pattern:
                entry[1] += 1
                return
        self.patterns.append([pattern, 1])


class FusionOptimizer:
    def __init__(self, config: FusionConfig | None = None):
        self.config = config or FusionConfig()
        self._stats = FusionStats()
        self.optimization_stats = OptimizationStats()

    @classmethod
    def new(cls): return cls()
    @classmethod
    def with_config(cls, config): return cls(config)

    def analyze(self, ops) -> list:
        ops = list(ops)
        pats = []
        for p, s, n in detect_patterns(ops):
            if p is FusionPattern.ElementwiseChain and (not self.config.fuse_elementwise or n < self.config.min_chain_length):
                continue
            if p.name.startswith("MatMul") and not self.config.fuse_linear: continue
            if p.name.startswith("Conv") and not self.config.fuse_conv: continue
            pats.append((p, s, n))
            self.optimization_stats.add_fusion(p, n)
        fused = sum(n for _, _, n in pats)
        self._stats = FusionStats(len(ops), fused, len(pats), estimate_speedup(ops, pats))
        return pats

    def stats(self) -> FusionStats: return self._stats

    def apply_fusions(self, patterns) -> None:
        """Counts ``(pattern, start, length)`` entries into ``optimization_stats`` (optimizer.rs:159-163)."""
        for p, _, n in patterns:
            self.optimization_stats.add_fusion(p, n)

    def reset_stats(self) -> None:
        self._stats = FusionStats()
        self.optimization_stats = OptimizationStats()


def estimate_speedup(ops, patterns) -> float:
    ops = list(ops)
    if not ops:
        return 1.0
    saved = sum(n * (1.0 - 1.0 / p.estimated_speedup()) for p, _, n in patterns)
    return len(ops) / max(len(ops) - saved, 1e-9)


def optimize_graph(ops, config: FusionConfig | None = None):
    opt = FusionOptimizer(config)
    return opt.analyze(ops), opt.stats()


def fold_conv_bn(conv: torch.nn.Module, bn: torch.nn.Module):
    """Returns ``(weight, bias)`` of the convolution equivalent to ``bn(conv(x))`` in eval mode."""
    w = conv.weight.detach().float()
    b = conv.bias.detach().float() if getattr(conv, "bias", None) is not None else torch.zeros(w.shape[0], device=w.device)
    scale = (bn.weight.detach().float() if bn.weight is not None else 1.0) / torch.sqrt(bn.running_var.float() + bn.eps)
    shift = (bn.bias.detach().float() if bn.bias is not None else 0.0) - bn.running_mean.float() * scale
    return w * scale.view(-1, *([1] * (w.dim() - 1))), b * scale + shift
