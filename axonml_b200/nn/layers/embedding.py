"""Embedding (crates/axonml-nn/src/layers/embedding.rs:40-103): ``weight[V,D]`` ~ N(0,1), the
``padding_idx`` row zeroed and excluded from gradients.  Indices may arrive as integer or (as in
the reference) float tensors."""
from __future__ import annotations

import torch

from ...ops import misc as _misc
from ..module import Module, Parameter


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None,
                 device=None, dtype=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        w = torch.randn(num_embeddings, embedding_dim)
        if padding_idx is not None:
            w[padding_idx] = 0
        self.weight = Parameter(w.to(device=device, dtype=dtype or torch.float32))

    @classmethod
    def new(cls, v, d): return cls(v, d)

    @classmethod
    def with_options(cls, v, d, padding_idx): return cls(v, d, padding_idx)

    @classmethod
    def from_pretrained(cls, weight: torch.Tensor, freeze: bool = True):
        m = cls(weight.shape[0], weight.shape[1])
        with torch.no_grad():
            m.weight.copy_(weight)
        m.weight.requires_grad_(not freeze)
        return m

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        if idx.is_floating_point():
            idx = idx.long()
        return _misc.embedding(idx, self.weight,
                               padding_idx=-1 if self.padding_idx is None else self.padding_idx)

    def lookup(self, indices: torch.Tensor) -> torch.Tensor:
        """``forward`` under the reference's name (embedding.rs:103-150).  An index outside the
        table raises ``IndexError`` (the reference clamps it to row 0 with a warning)."""
        idx = indices.long() if indices.is_floating_point() else indices
        if idx.numel() and (int(idx.max()) >= self.num_embeddings or int(idx.min()) < 0):
            raise IndexError(f"index out of range for a table of {self.num_embeddings} rows")
        return self.forward(idx)
