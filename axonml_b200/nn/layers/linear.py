"""Linear layer (crates/axonml-nn/src/layers/linear.rs:53-140): ``weight[out,in]`` drawn
kaiming-uniform with fan_in, zero bias, ``y = x W^T + b`` on any leading dims.  On a B200 in bf16
the forward and both backward GEMMs run on the tcgen05 kernel with bias/activation fused."""
from __future__ import annotations

import torch

from ...ops.linear import linear as _linear
from .. import init
from ..module import Module, Parameter


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 activation: str | None = None, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.activation = activation or "none"
        w = init.kaiming_uniform(out_features, in_features)
        self.weight = Parameter(w.to(device=device, dtype=dtype or torch.float32))
        if bias:
            self.bias = Parameter(torch.zeros(out_features, device=device, dtype=dtype or torch.float32))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, in_features: int, out_features: int) -> "Linear":
        return cls(in_features, out_features, True)

    @classmethod
    def with_bias(cls, in_features: int, out_features: int, bias: bool) -> "Linear":
        return cls(in_features, out_features, bias)

    @classmethod
    def from_weights(cls, weight: torch.Tensor, bias: torch.Tensor | None = None) -> "Linear":
        m = cls(weight.shape[1], weight.shape[0], bias is not None, dtype=weight.dtype,
                device=weight.device)
        with torch.no_grad():
            m.weight.copy_(weight)
            if bias is not None:
                m.bias.copy_(bias)
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _linear(x, self.weight, self.bias, self.activation)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"
