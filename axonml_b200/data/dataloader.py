"""DataLoader (crates/axonml-data/src/dataloader.rs:22-338): ``DataLoader.new(dataset, batch)``
with builders ``shuffle / drop_last / num_workers``; iteration yields ``Batch{data, targets,
size}``; indices are reshuffled per ``iter()``.  ``num_workers > 0`` fetches samples on a thread
pool, ``pin_memory`` and ``device`` stage batches through pinned host memory and copy them to the
GPU on a side stream one batch ahead of the consumer."""
from __future__ import annotations

import concurrent.futures as cf
import dataclasses

import torch

from .collate import DefaultCollate
from .sampler import BatchSampler, RandomSampler, SequentialSampler


@dataclasses.dataclass
class Batch:
    data: torch.Tensor
    targets: torch.Tensor
    size: int

    def len(self) -> int: return self.size
    def __len__(self) -> int: return self.size
    def is_empty(self) -> bool: return self.size == 0

    def to(self, device, non_blocking: bool = True) -> "Batch":
        return Batch(self.data.to(device, non_blocking=non_blocking),
                     self.targets.to(device, non_blocking=non_blocking), self.size)


class DataLoader:
    def __init__(self, dataset, batch_size: int = 1, shuffle: bool = False, drop_last: bool = False,
                 num_workers: int = 0, sampler=None, collate=None, pin_memory: bool = False, device=None):
        self.dataset, self.batch_size = dataset, batch_size
        self._shuffle, self._drop_last, self._num_workers = shuffle, drop_last, num_workers
        self._sampler, self._collate = sampler, collate or DefaultCollate()
        self._pin, self._device = pin_memory, device

    @classmethod
    def new(cls, dataset, batch_size: int): return cls(dataset, batch_size)
    def shuffle(self, flag: bool = True): self._shuffle = flag; return self
    def drop_last(self, flag: bool = True): self._drop_last = flag; return self
    def num_workers(self, n: int): self._num_workers = n; return self
    def sampler(self, s): self._sampler = s; return self
    def pin_memory(self, flag: bool = True): self._pin = flag; return self
    def to_device(self, device): self._device = device; return self

    def __len__(self) -> int:
        n = len(self._sampler) if self._sampler is not None else self.dataset.len()
        return n // self.batch_size if self._drop_last else (n + self.batch_size - 1) // self.batch_size

    def len(self) -> int: return len(self)
    def is_empty(self) -> bool: return len(self) == 0
    def dataset_len(self) -> int: return self.dataset.len()

    def _batches(self):
        base = self._sampler or (RandomSampler(self.dataset.len()) if self._shuffle else SequentialSampler(self.dataset.len()))
        return BatchSampler(base, self.batch_size, self._drop_last)

    def _make(self, indices, pool):
        samples = list(pool.map(self.dataset.get, indices)) if pool else [self.dataset.get(i) for i in indices]
        out = self._collate(samples)
        data, targets = out if isinstance(out, tuple) and len(out) == 2 else (out, torch.empty(0))
        if self._pin and torch.cuda.is_available():
            data, targets = data.pin_memory(), targets.pin_memory()
        return Batch(data, targets, len(indices))

    def iter(self): return DataLoaderIter(self)

    def __iter__(self):
        pool = cf.ThreadPoolExecutor(self._num_workers) if self._num_workers > 0 else None
        try:
            if self._device is None or not torch.cuda.is_available():
                for idx in self._batches():
                    yield self._make(idx, pool)
                return
            # one-batch-ahead prefetch to the device on a copy stream
            stream = torch.cuda.Stream()
            nxt = None
            for idx in self._batches():
                b = self._make(idx, pool)
                with torch.cuda.stream(stream):
                    staged = b.to(self._device)
                    ev = torch.cuda.Event()
                    ev.record(stream)
                if nxt is not None:
                    torch.cuda.current_stream().wait_event(nxt[1])
                    yield nxt[0]
                nxt = (staged, ev)
            if nxt is not None:
                torch.cuda.current_stream().wait_event(nxt[1])
                yield nxt[0]
        finally:
            if pool:
                pool.shutdown(wait=False)


class DataLoaderIter:
    """One pass over a loader (dataloader.rs:160-225): an iterator that also knows how many batches
    are left.  The index order is drawn when the iterator is created, so two iterators of a
    shuffling loader see different orders."""

    def __init__(self, loader: DataLoader):
        self.loader = loader
        self.position = 0                   # batches handed out so far
        self._total = len(loader)
        self._it = loader.__iter__()

    def __iter__(self): return self

    def __next__(self):
        b = next(self._it)
        self.position += 1
        return b

    def next(self):
        """The next batch, or ``None`` after the last one."""
        try:
            return self.__next__()
        except StopIteration:
            return None

    def remaining(self) -> int: return max(self._total - self.position, 0)
    def __len__(self) -> int: return self.remaining()


class GenericDataLoader(DataLoader):
    """DataLoader over datasets whose samples are not (tensor, tensor) pairs; yields whatever the
    collate function returns."""

    def _make(self, indices, pool):
        samples = list(pool.map(self.dataset.get, indices)) if pool else [self.dataset.get(i) for i in indices]
        return self._collate(samples)

    def iter(self): return GenericDataLoaderIter(self)


class GenericDataLoaderIter(DataLoaderIter):
    """One pass over a ``GenericDataLoader`` (dataloader.rs ``GenericDataLoaderIter``): yields what
    the loader's collate function returns."""
