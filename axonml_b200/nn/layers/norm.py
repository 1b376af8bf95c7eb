"""Normalisation layers (crates/axonml-nn/src/layers/norm.rs): BatchNorm1d/2d (eps 1e-5,
momentum 0.1, biased batch variance, running = (1-m)*running + m*batch as in norm.rs:339-357),
LayerNorm, GroupNorm, InstanceNorm2d.  Running statistics are registered buffers so that they
are serialised (the reference keeps them private and loses them on save)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import norm as _norm
from ..module import Module, Parameter


class _BatchNorm(Module):
    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1,
                 affine: bool = True, track_running_stats: bool = True):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.affine, self.track_running_stats = affine, track_running_stats
        if affine:
            self.weight = Parameter(torch.ones(num_features))
            self.bias = Parameter(torch.zeros(num_features))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self.register_buffer("running_mean", torch.zeros(num_features))
        self.register_buffer("running_var", torch.ones(num_features))
        self.register_buffer("num_batches_tracked", torch.zeros((), dtype=torch.long))

    @classmethod
    def new(cls, num_features): return cls(num_features)

    @classmethod
    def with_options(cls, num_features, eps, momentum, affine=True): return cls(num_features, eps, momentum, affine)

    def forward(self, x, relu: bool = False, residual=None):
        """``relu`` / ``residual`` fuse the block's activation and skip connection into the
        normalisation pass (one kernel on channels-last bf16 inputs)."""
        use_batch = self.training or not self.track_running_stats
        if x.dim() == 4:
            from ...ops import batchnorm as BN
            if use_batch and self.track_running_stats:
                with torch.no_grad():
                    self.num_batches_tracked += 1
            return BN.batch_norm(x, self.weight, self.bias,
                                 self.running_mean if self.track_running_stats else None,
                                 self.running_var if self.track_running_stats else None,
                                 use_batch, self.momentum, self.eps, relu, residual)
        if use_batch and self.track_running_stats:
            # the reference updates running_var with the biased batch variance
            with torch.no_grad():
                dims = [0] + list(range(2, x.dim()))
                xf = x.detach().float()
                mean = xf.mean(dims)
                var = xf.var(dims, unbiased=False)
                self.running_mean.mul_(1 - self.momentum).add_(mean, alpha=self.momentum)
                self.running_var.mul_(1 - self.momentum).add_(var, alpha=self.momentum)
                self.num_batches_tracked += 1
            y = F.batch_norm(x, None, None, self.weight, self.bias, True, 0.0, self.eps)
        else:
            y = F.batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias,
                             use_batch, 0.0, self.eps)
        if residual is not None:
            y = y + residual
        return torch.relu(y) if relu else y


class BatchNorm1d(_BatchNorm):
    pass


class BatchNorm2d(_BatchNorm):
    pass


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        n = 1
        for s in self.normalized_shape:
            n *= s
        self._n = n
        self.weight = Parameter(torch.ones(self.normalized_shape, device=device, dtype=dtype or torch.float32))
        self.bias = Parameter(torch.zeros(self.normalized_shape, device=device, dtype=dtype or torch.float32))

    @classmethod
    def new(cls, shape): return cls(shape)

    @classmethod
    def single(cls, n: int): return cls((n,))

    @classmethod
    def with_eps(cls, shape, eps: float): return cls(shape, eps)

    def forward(self, x, residual=None):
        if len(self.normalized_shape) == 1:
            w, b = self.weight, self.bias
            if x.dtype == torch.bfloat16 and w.dtype not in (torch.bfloat16, torch.float32):
                w, b = w.float(), b.float()
            return _norm.layer_norm(x, w, b, self.eps, residual=residual)
        lead = x.shape[: x.dim() - len(self.normalized_shape)]
        y = _norm.layer_norm(x.reshape(*lead, self._n), self.weight.reshape(-1), self.bias.reshape(-1), self.eps)
        return y.reshape(x.shape)


class RMSNorm(Module):
    """``x * rsqrt(mean(x^2) + eps) * weight`` (crates/axonml-llm/src/llama.rs:138-198)."""

    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = Parameter(torch.ones(dim, device=device, dtype=dtype or torch.float32))

    @classmethod
    def new(cls, dim: int, eps: float = 1e-5): return cls(dim, eps)

    def forward(self, x, residual=None):
        return _norm.rms_norm(x, self.weight, self.eps, residual=residual)

    def load_weight(self, weight) -> None:
        """Replaces the scale vector (llama.rs ``RMSNorm::load_weight``)."""
        w = torch.as_tensor(weight)
        if w.shape != self.weight.shape:
            raise ValueError(f"expected shape {tuple(self.weight.shape)}, got {tuple(w.shape)}")
        with torch.no_grad():
            self.weight.copy_(w.to(self.weight.dtype))


class GroupNorm(Module):
    def __init__(self, num_groups: int, num_channels: int, eps: float = 1e-5, affine: bool = True):
        super().__init__()
        self.num_groups, self.num_channels, self.eps, self.affine = num_groups, num_channels, eps, affine
        if affine:
            self.weight = Parameter(torch.ones(num_channels))
            self.bias = Parameter(torch.zeros(num_channels))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, groups, channels): return cls(groups, channels)

    @classmethod
    def with_options(cls, groups, channels, eps, affine): return cls(groups, channels, eps, affine)

    def forward(self, x):
        return F.group_norm(x, self.num_groups, self.weight, self.bias, self.eps)


class InstanceNorm2d(Module):
    def __init__(self, num_features: int, eps: float = 1e-5, affine: bool = False):
        super().__init__()
        self.num_features, self.eps, self.affine = num_features, eps, affine
        if affine:
            self.weight = Parameter(torch.ones(num_features))
            self.bias = Parameter(torch.zeros(num_features))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, c): return cls(c)

    @classmethod
    def with_affine(cls, c): return cls(c, affine=True)

    @classmethod
    def with_options(cls, c, eps, affine): return cls(c, eps, affine)

    def forward(self, x):
        return F.instance_norm(x, None, None, self.weight, self.bias, True, 0.0, self.eps)
