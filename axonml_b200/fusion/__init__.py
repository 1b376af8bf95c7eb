"""Operator fusion (crates/axonml-fusion)."""
from .ops import (Activation, ElementwiseOp, FusedElementwise, FusedElementwiseBuilder, FusedLinear, FusedOp, FusionError,
                  fuse_elementwise, fuse_linear, fuse_matmul_bias, fuse_matmul_bias_gelu, fuse_matmul_bias_relu, fused_add_relu,
                  fused_elementwise, fused_mul_add, fused_scale_bias_relu)
from .patterns import (FusionConfig, FusionOptimizer, FusionPattern, FusionStats, OptimizationStats, OpType, detect_patterns,
                       estimate_speedup, fold_conv_bn, optimize_graph)
