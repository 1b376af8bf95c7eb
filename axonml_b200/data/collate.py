"""Collation (crates/axonml-data/src/collate.rs): ``stack_tensors``, ``DefaultCollate``,
``StackCollate`` and the ``Collate`` protocol."""
from __future__ import annotations

import torch


def stack_tensors(tensors):
    return torch.stack([torch.as_tensor(t) for t in tensors], 0)


def concat_tensors(tensors, dim: int = 0):
    return torch.cat(list(tensors), dim)


class Collate:
    def collate(self, samples): raise NotImplementedError
    def __call__(self, samples): return self.collate(samples)


class DefaultCollate(Collate):
    def collate(self, samples):
        first = samples[0]
        if isinstance(first, (tuple, list)):
            return tuple(stack_tensors([s[i] for s in samples]) for i in range(len(first)))
        return stack_tensors(samples)


class StackCollate(Collate):
    def __init__(self, dim: int = 0): self.dim = dim
    @classmethod
    def new(cls): return cls(0)
    @classmethod
    def with_dim(cls, dim: int): return cls(dim)
    def collate(self, samples): return torch.stack(list(samples), self.dim)
