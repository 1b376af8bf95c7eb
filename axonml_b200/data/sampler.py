"""Samplers (crates/axonml-data/src/sampler.rs:18-323) plus ``DistributedSampler``, which the
reference lacks: each rank takes every world-th index of a per-epoch seeded permutation."""
from __future__ import annotations

import math

import torch


class Sampler:
    def __iter__(self): raise NotImplementedError
    def __len__(self): raise NotImplementedError
    def len(self): return len(self)


class SequentialSampler(Sampler):
    def __init__(self, n: int): self.n = n
    def __iter__(self): return iter(range(self.n))
    def __len__(self): return self.n


class RandomSampler(Sampler):
    def __init__(self, n: int, replacement: bool = False, num_samples: int | None = None, generator=None):
        self.n, self.replacement, self.num_samples, self.generator = n, replacement, num_samples or n, generator

    @classmethod
    def with_replacement(cls, n, num_samples): return cls(n, True, num_samples)

    def __iter__(self):
        if self.replacement:
            return iter(torch.randint(0, self.n, (self.num_samples,), generator=self.generator).tolist())
        return iter(torch.randperm(self.n, generator=self.generator).tolist()[: self.num_samples])

    def __len__(self): return self.num_samples


class SubsetRandomSampler(Sampler):
    def __init__(self, indices, generator=None): self.indices, self.generator = list(indices), generator
    def __iter__(self):
        return iter(self.indices[i] for i in torch.randperm(len(self.indices), generator=self.generator).tolist())
    def __len__(self): return len(self.indices)


class WeightedRandomSampler(Sampler):
    def __init__(self, weights, num_samples: int, replacement: bool = True, generator=None):
        self.weights = torch.as_tensor(weights, dtype=torch.float64)
        self.num_samples, self.replacement, self.generator = num_samples, replacement, generator

    def __iter__(self):
        return iter(torch.multinomial(self.weights, self.num_samples, self.replacement, generator=self.generator).tolist())

    def __len__(self): return self.num_samples


class BatchIter:
    """Iterator over lists of indices, ``batch_size`` at a time (sampler.rs:323-348); a short last
    batch is dropped when ``drop_last``."""

    def __init__(self, indices, batch_size: int, drop_last: bool = False):
        if batch_size <= 0:
            raise ValueError("batch_size must be positive")
        self.indices, self.batch_size, self.drop_last, self.position = list(indices), batch_size, drop_last, 0

    def __iter__(self): return self

    def __next__(self) -> list:
        if self.position >= len(self.indices):
            raise StopIteration
        batch = self.indices[self.position:self.position + self.batch_size]
        if len(batch) < self.batch_size and self.drop_last:
            self.position = len(self.indices)
            raise StopIteration
        self.position += len(batch)
        return batch

    def remaining(self) -> int:
        left = len(self.indices) - self.position
        return left // self.batch_size if self.drop_last else -(-left // self.batch_size)


class BatchSampler(Sampler):
    def __init__(self, sampler: Sampler, batch_size: int, drop_last: bool = False):
        self.sampler, self.batch_size, self.drop_last = sampler, batch_size, drop_last

    def __iter__(self):
        return BatchIter(self.sampler, self.batch_size, self.drop_last)

    iter = __iter__

    def __len__(self):
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else math.ceil(n / self.batch_size)

    def len(self) -> int: return len(self)
    def is_empty(self) -> bool: return len(self) == 0


class DistributedSampler(Sampler):
    def __init__(self, n: int, world_size: int, rank: int, shuffle: bool = True, seed: int = 0,
                 drop_last: bool = False):
        self.n, self.world, self.rank, self.shuffle, self.seed, self.drop_last = n, world_size, rank, shuffle, seed, drop_last
        self.epoch = 0
        self.per_rank = n // world_size if drop_last else math.ceil(n / world_size)

    def set_epoch(self, epoch: int) -> None: self.epoch = epoch

    def __iter__(self):
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            idx = torch.randperm(self.n, generator=g).tolist()
        else:
            idx = list(range(self.n))
        total = self.per_rank * self.world
        if self.drop_last:
            idx = idx[:total]
        else:
            idx += idx[: total - len(idx)]
        return iter(idx[self.rank:total:self.world])

    def __len__(self): return self.per_rank
