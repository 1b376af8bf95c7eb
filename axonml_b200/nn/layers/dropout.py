"""Dropout layers (crates/axonml-nn/src/layers/dropout.rs:26-118), inverted scaling."""
from __future__ import annotations

import torch.nn.functional as F

from ...ops import elementwise as E
from ..module import Module


class Dropout(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        if not 0.0 <= p < 1.0:
            raise ValueError("dropout probability must be in [0, 1)")
        self.p = p

    @classmethod
    def new(cls, p: float): return cls(p)

    @classmethod
    def default_p(cls): return cls(0.5)

    def forward(self, x): return E.dropout(x, self.p, self.training)


class Dropout2d(Dropout):
    def forward(self, x): return F.dropout2d(x, self.p, self.training)


class AlphaDropout(Dropout):
    def forward(self, x): return F.alpha_dropout(x, self.p, self.training)
