"""Reference-counted storage with offset/length views (crates/axonml-core/src/storage.rs:43-236)
and allocators (allocator.rs).  A ``Storage`` wraps a flat torch tensor, so views share memory and
``to_device`` works for CUDA as well (the reference refuses every non-CPU device,
storage.rs:224-235).  ``CachingDeviceAllocator`` pools device segments and carves them with the
native offset allocator (``csrc/host/arena.cpp``, ``OffsetArena``), which the symmetric heap of the
fused collectives uses too."""
from __future__ import annotations

import threading

import torch

from .device import Device, as_torch_device
from .dtype import as_torch_dtype
from .error import AllocationFailed, DeviceNotAvailable, IndexOutOfBounds


class _RwLock:
    """Many readers or one writer; shared by every view of one buffer."""

    def __init__(self):
        self._cond = threading.Condition()
        self._readers = 0
        self._writer = False

    def acquire_read(self, timeout=None) -> bool:
        with self._cond:
            if not self._cond.wait_for(lambda: not self._writer, timeout):
                return False
            self._readers += 1
            return True

    def release_read(self) -> None:
        with self._cond:
            self._readers -= 1
            if self._readers == 0:
                self._cond.notify_all()

    def acquire_write(self, timeout=None) -> bool:
        with self._cond:
            if not self._cond.wait_for(lambda: not self._writer and self._readers == 0, timeout):
                return False
            self._writer = True
            return True

    def release_write(self) -> None:
        with self._cond:
            self._writer = False
            self._cond.notify_all()


class _Guard:
    def __init__(self, storage, timeout):
        self._storage, self._live = storage, True
        if not self._acquire(storage._lock, timeout):
            self._live = False
            raise TimeoutError("storage is locked")

    def tensor(self) -> torch.Tensor:
        """The guarded elements (a view; valid until the guard is dropped)."""
        if not self._live:
            raise RuntimeError("the guard has been dropped")
        return self._storage.as_tensor()

    def __len__(self) -> int: return self._storage.len()
    def __getitem__(self, i): return self.tensor()[i]
    def to_vec(self) -> list: return self.tensor().tolist()

    def drop(self) -> None:
        if self._live:
            self._live = False
            self._release(self._storage._lock)

    def __enter__(self): return self
    def __exit__(self, *exc): self.drop()
    def __del__(self): self.drop()


class StorageReadGuard(_Guard):
    """Shared access to a storage's elements (storage.rs:253-266): any number at a time, none while
    a write guard is held."""
    _acquire = staticmethod(_RwLock.acquire_read)
    _release = staticmethod(_RwLock.release_read)


class StorageWriteGuard(_Guard):
    """Exclusive access (storage.rs:268-290): waits for every other guard of the buffer to be dropped."""
    _acquire = staticmethod(_RwLock.acquire_write)
    _release = staticmethod(_RwLock.release_write)

    def __setitem__(self, i, value): self.tensor()[i] = value
    def fill(self, value) -> None: self.tensor().fill_(value)
    def copy_from(self, values) -> None: self.tensor().copy_(torch.as_tensor(values, dtype=self.tensor().dtype))


class Storage:
    def __init__(self, data: torch.Tensor, offset: int = 0, length: int | None = None, _lock: _RwLock | None = None):
        self._base = data.reshape(-1)
        self._offset = offset
        self._len = self._base.numel() - offset if length is None else length
        self._lock = _lock or _RwLock()               # views made with slice() share it

    def read(self, timeout: float | None = None) -> StorageReadGuard:
        """Read guard (``as_slice`` of the reference): ``with st.read() as r: r.tensor()``."""
        return StorageReadGuard(self, timeout)

    def write(self, timeout: float | None = None) -> StorageWriteGuard:
        """Write guard (``as_slice_mut`` of the reference)."""
        return StorageWriteGuard(self, timeout)

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
        return Storage(self._base, self._offset + offset, length, self._lock)

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


class OffsetArena:
    """Native offset allocator over ``[0, capacity)`` (``csrc/host/arena.cpp``): best fit with
    splitting, neighbours merged on free, deterministic.  It never touches memory; the caller owns
    the range the offsets refer to."""

    def __init__(self, capacity: int, alignment: int = 512):
        import ctypes
        from .. import _native as N
        self._lib = N.host()
        self._lib.ax_arena_create.restype = ctypes.c_void_p
        self._lib.ax_arena_alloc.restype = ctypes.c_int64
        self._lib.ax_arena_block_size.restype = ctypes.c_uint64
        self._h = self._lib.ax_arena_create(ctypes.c_uint64(capacity), ctypes.c_uint64(alignment))
        if not self._h:
            raise ValueError("capacity must be positive and the alignment a power of two")
        self.alignment = alignment

    def alloc(self, nbytes: int) -> int:
        """Offset of a block of at least ``nbytes`` bytes, or -1."""
        import ctypes
        return int(self._lib.ax_arena_alloc(ctypes.c_void_p(self._h), ctypes.c_uint64(nbytes)))

    def free(self, offset: int) -> bool:
        import ctypes
        return self._lib.ax_arena_free(ctypes.c_void_p(self._h), ctypes.c_int64(offset)) == 0

    def block_size(self, offset: int) -> int:
        import ctypes
        return int(self._lib.ax_arena_block_size(ctypes.c_void_p(self._h), ctypes.c_int64(offset)))

    def reset(self) -> None:
        import ctypes
        self._lib.ax_arena_reset(ctypes.c_void_p(self._h))

    def stats(self) -> dict:
        import ctypes
        out = (ctypes.c_uint64 * 7)()
        self._lib.ax_arena_stats(ctypes.c_void_p(self._h), out)
        keys = ("capacity", "in_use", "peak", "live_blocks", "free_blocks", "largest_free", "allocations")
        return dict(zip(keys, (int(v) for v in out)))

    def __del__(self):
        try:
            import ctypes
            if getattr(self, "_h", None):
                self._lib.ax_arena_destroy(ctypes.c_void_p(self._h))
                self._h = None
        except Exception:
            pass


class CachingDeviceAllocator(Allocator):
    """Pool allocator for runtime buffers that are reused across steps (communication staging,
    kernel scratch): memory comes from the device in segments of ``segment_bytes`` (one driver call
    each) and the native offset allocator carves tensors out of them, so the steady state of a
    training loop makes no driver calls.  Requests larger than a segment get a segment of their own.
    ``deallocate`` returns a block to its segment (neighbouring free blocks merge); ``empty_cache``
    releases the segments that hold no live block."""

    def __init__(self, device=None, round_to: int = 512, segment_bytes: int = 64 << 20):
        self.dev = device or (Device.Cuda(torch.cuda.current_device()) if torch.cuda.is_available() else Device.Cpu())
        self.round_to, self.segment_bytes = round_to, segment_bytes
        self._segments: list[tuple[torch.Tensor, OffsetArena]] = []
        self._owner: dict[int, tuple[int, int]] = {}          # data_ptr -> (segment index, offset)
        self._lock = threading.Lock()
        self.hits = self.misses = 0                           # served from a cached segment / needed a new one

    def _new_segment(self, nbytes: int):
        size = max(self.segment_bytes, (nbytes + self.round_to - 1) // self.round_to * self.round_to)
        try:
            raw = torch.empty(size + self.round_to, dtype=torch.uint8, device=self.dev.to_torch())
        except RuntimeError as e:
            raise AllocationFailed(size, str(self.dev)) from e
        shift = (-raw.data_ptr()) % self.round_to          # blocks are aligned in memory, not only inside the segment
        raw = raw[shift:shift + size]
        seg = (raw, OffsetArena(size, self.round_to))
        for i, s in enumerate(self._segments):
            if s is None:
                self._segments[i] = seg
                return i
        self._segments.append(seg)
        return len(self._segments) - 1

    def allocate(self, count: int, dtype=torch.float32):
        dt = as_torch_dtype(dtype)
        nbytes = max(1, count * torch.empty((), dtype=dt).element_size())
        with self._lock:
            idx, off = -1, -1
            for i, seg in enumerate(self._segments):
                if seg is None:
                    continue
                off = seg[1].alloc(nbytes)
                if off >= 0:
                    idx = i
                    self.hits += 1
                    break
            if idx < 0:
                self.misses += 1
                idx = self._new_segment(nbytes)
                off = self._segments[idx][1].alloc(nbytes)
            raw = self._segments[idx][0]
            t = raw[off:off + nbytes].view(dt)[:count]
            self._owner[t.data_ptr()] = (idx, off)
        return t

    def deallocate(self, t) -> None:
        with self._lock:
            where = self._owner.pop(t.data_ptr(), None)
            if where is not None:
                self._segments[where[0]][1].free(where[1])

    def empty_cache(self) -> None:
        with self._lock:
            for i, seg in enumerate(self._segments):
                if seg is not None and seg[1].stats()["live_blocks"] == 0:
                    self._segments[i] = None

    def total_memory(self) -> int: return self.dev.capabilities().total_memory
    def free_memory(self) -> int: return self.dev.capabilities().available_memory

    def cached_bytes(self) -> int:
        """Bytes held in segments but not handed out."""
        with self._lock:
            return sum(s[1].stats()["capacity"] - s[1].stats()["in_use"] for s in self._segments if s is not None)

    def stats(self) -> dict:
        with self._lock:
            segs = [s[1].stats() for s in self._segments if s is not None]
        return {"segments": len(segs), "reserved": sum(s["capacity"] for s in segs), "in_use": sum(s["in_use"] for s in segs),
                "peak": sum(s["peak"] for s in segs), "live_blocks": sum(s["live_blocks"] for s in segs),
                "hits": self.hits, "misses": self.misses}
