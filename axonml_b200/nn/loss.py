"""Loss modules (crates/axonml-nn/src/loss.rs:19-452).  Every loss is constructed with
``new()`` (mean reduction) or ``with_reduction(Reduction)`` and evaluated with
``.compute(input, target)`` (also callable).  Targets of CrossEntropy/NLL are class indices and
may be float tensors as in the reference.  All losses are differentiable (the reference's
CrossEntropy/NLL cut the graph, loss.rs:196-197)."""
from __future__ import annotations

import enum

import torch
import torch.nn.functional as F

from ..ops import loss as L
from .module import Module


class Reduction(enum.Enum):
    None_ = "none"
    Mean = "mean"
    Sum = "sum"


Reduction.NONE = Reduction.None_


def _red(r) -> str:
    if isinstance(r, Reduction):
        return r.value
    return {"none": "none", "mean": "mean", "sum": "sum"}[str(r).lower()]


class _Loss(Module):
    def __init__(self, reduction=Reduction.Mean):
        super().__init__()
        self.reduction = _red(reduction)

    @classmethod
    def new(cls): return cls()

    @classmethod
    def with_reduction(cls, reduction): return cls(reduction)

    def forward(self, input, target): return self.compute(input, target)


class MSELoss(_Loss):
    def compute(self, input, target): return F.mse_loss(input, target, reduction=self.reduction)


class L1Loss(_Loss):
    def compute(self, input, target): return F.l1_loss(input, target, reduction=self.reduction)


class CrossEntropyLoss(_Loss):
    def __init__(self, reduction=Reduction.Mean, ignore_index: int = -100):
        super().__init__(reduction)
        self.ignore_index = ignore_index

    def compute(self, input, target):
        if target.is_floating_point() and target.dim() == input.dim():
            return F.cross_entropy(input, target, reduction=self.reduction)  # class probabilities
        if target.is_floating_point():
            target = target.long()
        return L.cross_entropy(input, target, ignore_index=self.ignore_index, reduction=self.reduction)


class NLLLoss(_Loss):
    def compute(self, input, target):
        return F.nll_loss(input, target.long(), reduction=self.reduction)


class BCELoss(_Loss):
    def compute(self, input, target):
        return F.binary_cross_entropy(input, target, reduction=self.reduction)


class BCEWithLogitsLoss(_Loss):
    def compute(self, input, target):
        return F.binary_cross_entropy_with_logits(input, target, reduction=self.reduction)


class SmoothL1Loss(_Loss):
    def __init__(self, reduction=Reduction.Mean, beta: float = 1.0):
        super().__init__(reduction)
        self.beta = beta

    @classmethod
    def with_beta(cls, beta: float): return cls(beta=beta)

    def compute(self, input, target):
        return F.smooth_l1_loss(input, target, reduction=self.reduction, beta=self.beta)
