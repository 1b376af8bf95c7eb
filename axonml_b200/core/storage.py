"""Reference-counted storage with offset/length views (crates/axonml-core/src/storage.rs:43-236)
and allocators (allocator.rs).  A ``Storage`` wraps a flat torch tensor, so views share memory and
``to_device`` works for CUDA as well (the reference refuses every non-CPU device,
storage.rs:224-235).  ``CachingDeviceAllocator`` is a size-bucketed free list on top of
``torch.empty`` for runtime buffers that are reused across steps (communication staging, kernel
scratch) without going back to the driver."""
from __future__ import annotations

import collections
import threading

import torch

from .device import Device, as_torch_device
from .dtype import as_torch_dtype
from .error import AllocationFailed, DeviceNotAvailable, IndexOutOfBounds


class Storage:
    def __init__(self, data: torch.Tensor, offset: int = 0, length: int | None = None):
        self._base = data.reshape(-1)
        self._offset = offset
        self._len = self._base.numel() - offset if length is None else length

    @classmethod
    def zeros(cls, length: int, device=Device.Cpu(), dtype=torch.float32):
        return cls(torch.zeros(length, dtype=as_torch_dtype(dtype), device=as_torch_device(device)))

    @classmethod
    def from_vec(cls, data, device=Device.Cpu(), dtype=torch.float32):
        return cls(torch.tensor(data, dtype=as_torch_dtype(dtype), device=as_torch_device(device)))

    from_slice = from_vec

    def len(self) -> int: return self._len
    def __len__(self) -> int: return self._len
    def is_empty(self) -> bool: return self._len == 0
    def offset(self) -> int: return self._offset
    def device(self) -> Device: return Device.from_torch(self._base.device)
    def size_bytes(self) -> int: return self._len * self._base.element_size()
    def as_tensor(self) -> torch.Tensor: return self._base[self._offset:self._offset + self._len]
    as_slice = as_tensor
    as_slice_mut = as_tensor

    def slice(self, offset: int, length: int) -> "Storage":
        if offset + length > self._len:
            raise IndexOutOfBounds(offset + length, self._len)
        return Storage(self._base, self._offset + offset, length)

    def is_unique(self) -> bool:
        import sys
        return sys.getrefcount(self._base) <= 3

    def copy_from(self, other: "Storage") -> None:
        if other.len() != self._len:
            raise IndexOutOfBounds(other.len(), self._len)
        self.as_tensor().copy_(other.as_tensor())

    def deep_copy(self) -> "Storage": return Storage(self.as_tensor().clone())

    def to_device(self, device) -> "Storage":
        dev = device if isinstance(device, Device) else Device.from_torch(device)
        if not dev.is_available():
            raise DeviceNotAvailable(str(dev))
        return Storage(self.as_tensor().to(dev.to_torch()))


class Allocator:
    def allocate(self, count: int, dtype=torch.float32): raise NotImplementedError
    def deallocate(self, t) -> None: pass
    def total_memory(self) -> int: raise NotImplementedError
    def free_memory(self) -> int: raise NotImplementedError


class DefaultAllocator(Allocator):
    def __init__(self, device=Device.Cpu()): self.dev = device

    def allocate(self, count: int, dtype=torch.float32):
        try:
            return torch.empty(count, dtype=as_torch_dtype(dtype), device=self.dev.to_torch())
        except RuntimeError as e:
            raise AllocationFailed(count, str(self.dev)) from e

    def total_memory(self) -> int: return self.dev.capabilities().total_memory
    def free_memory(self) -> int: return self.dev.capabilities().available_memory


class CachingDeviceAllocator(Allocator):
    def __init__(self, device=None, round_to: int = 512):
        self.dev = device or (Device.Cuda(torch.cuda.current_device()) if torch.cuda.is_available() else Device.Cpu())
        self.round_to = round_to
        self._free = collections.defaultdict(list)
        self._lock = threading.Lock()
        self.hits = self.misses = 0

    def _bucket(self, nbytes: int) -> int:
        return (nbytes + self.round_to - 1) // self.round_to * self.round_to

    def allocate(self, count: int, dtype=torch.float32):
        dt = as_torch_dtype(dtype)
        nbytes = self._bucket(count * torch.empty((), dtype=dt).element_size())
        with self._lock:
            lst = self._free.get(nbytes)
            if lst:
                self.hits += 1
                raw = lst.pop()
            else:
                self.misses += 1
                raw = None
        if raw is None:
            try:
                raw = torch.empty(nbytes, dtype=torch.uint8, device=self.dev.to_torch())
            except RuntimeError as e:
                raise AllocationFailed(nbytes, str(self.dev)) from e
        t = raw.view(dt)[:count]
        t._axon_raw = raw
        return t

    def deallocate(self, t) -> None:
        raw = getattr(t, "_axon_raw", None)
        if raw is not None:
            with self._lock:
                self._free[raw.numel()].append(raw)

    def empty_cache(self) -> None:
        with self._lock:
            self._free.clear()

    def total_memory(self) -> int: return self.dev.capabilities().total_memory
    def free_memory(self) -> int: return self.dev.capabilities().available_memory
    def cached_bytes(self) -> int: return sum(k * len(v) for k, v in self._free.items())
