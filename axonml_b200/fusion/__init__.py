"""Operator fusion (crates/axonml-fusion)."""
from .ops import (Activation, ElementwiseOp, FusedElementwise, FusedElementwiseBuilder, FusedLinear, FusedOp,
                  fuse_linear, fused_elementwise)
from .patterns import (FusionConfig, FusionOptimizer, FusionPattern, FusionStats, OpType, detect_patterns,
                       estimate_speedup, fold_conv_bn, optimize_graph)
