"""Datasets (crates/axonml-data/src/dataset.rs:17-287): ``Dataset{len,get}``, TensorDataset,
MapDataset, ConcatDataset, SubsetDataset (+``random_split``), InMemoryDataset."""
from __future__ import annotations

import torch


class Dataset:
    def len(self) -> int: raise NotImplementedError
    def get(self, index: int): raise NotImplementedError
    def __len__(self) -> int: return self.len()

    def __getitem__(self, index: int):
        """``dataset[i]`` with Python's conventions: negative positions count from the end and a
        position past the end raises ``IndexError`` (which also ends ``for sample in dataset``)."""
        n = self.len()
        if index < 0:
            index += n
        if not 0 <= index < n:
            raise IndexError(f"index {index} out of range for a dataset of {n} samples")
        return self.get(index)

    def is_empty(self) -> bool: return self.len() == 0


class TensorDataset(Dataset):
    def __init__(self, data: torch.Tensor, targets: torch.Tensor):
        if data.shape[0] != targets.shape[0]:
            raise ValueError("data and targets differ in length")
        self.data, self.targets = data, targets

    @classmethod
    def new(cls, data, targets): return cls(data, targets)

    @classmethod
    def from_data(cls, data: torch.Tensor):
        """Unlabelled data: every target is 0 (dataset.rs:66-70)."""
        return cls(data, torch.zeros(data.shape[0]))

    def len(self) -> int: return self.data.shape[0]
    def get(self, index: int): return self.data[index], self.targets[index]


class MapDataset(Dataset):
    def __init__(self, dataset: Dataset, fn):
        self.dataset, self.fn = dataset, fn

    def len(self) -> int: return self.dataset.len()
    def get(self, index: int): return self.fn(*self.dataset.get(index))


class ConcatDataset(Dataset):
    def __init__(self, datasets):
        self.datasets = list(datasets)
        self._cum = []
        total = 0
        for d in self.datasets:
            total += d.len()
            self._cum.append(total)

    def len(self) -> int: return self._cum[-1] if self._cum else 0

    def get(self, index: int):
        prev = 0
        for d, c in zip(self.datasets, self._cum):
            if index < c:
                return d.get(index - prev)
            prev = c
        raise IndexError(index)


class SubsetDataset(Dataset):
    def __init__(self, dataset: Dataset, indices):
        self.dataset, self.indices = dataset, list(indices)

    def len(self) -> int: return len(self.indices)
    def get(self, index: int): return self.dataset.get(self.indices[index])

    @staticmethod
    def random_split(dataset: Dataset, lengths, generator=None):
        n = dataset.len()
        if sum(lengths) != n:
            raise ValueError("split lengths must sum to the dataset length")
        perm = torch.randperm(n, generator=generator).tolist()
        out, off = [], 0
        for length in lengths:
            out.append(SubsetDataset(dataset, perm[off:off + length]))
            off += length
        return out


random_split = SubsetDataset.random_split


class InMemoryDataset(Dataset):
    def __init__(self, samples):
        self.samples = list(samples)

    def len(self) -> int: return len(self.samples)
    def get(self, index: int): return self.samples[index]
    def push(self, sample) -> None: self.samples.append(sample)
