"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

``SymmetricHeap.allocate`` returns a buffer that exists at the same size on every rank of a
process group, is mapped into every peer's address space (all GPUs of a B200 box reach each other
at full bandwidth through NVSwitch, so no topology logic is needed) and, when the driver offers
it, is also bound to an NVLS multicast address for ``multimem`` instructions.  The rendezvous
(exchange of handles between processes) is done by ``torch.distributed._symmetric_memory``; what
runs on the buffers are this package's own kernels.

``AXONML_NVLS=0`` disables the multicast mapping (kernels then use plain peer loads/stores); the
failure-detection tests run that way.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native as N


def available(pg) -> bool:
    if not (torch.cuda.is_available() and dist.is_initialized() and pg.world_size() > 1):
        return False
    try:
        import importlib
        importlib.import_module("torch.distributed._symmetric_memory")
        return True
    except Exception:
        return False


class SymmetricBuffer:
    """One symmetric allocation: ``local`` (this rank's tensor), peer pointers, multicast pointer."""

    def __init__(self, local: torch.Tensor, handle, use_mc: bool):
        self.local = local
        self.handle = handle
        self.world = handle.world_size
        self.rank = handle.rank
        self.peer_ptrs = [int(p) for p in handle.buffer_ptrs]
        mc = 0
        if use_mc:
            try:
                mc = int(handle.multicast_ptr) if handle.has_multicast_support() else 0
            except Exception:
                mc = 0
        self.mc_ptr = mc
        self._arr = (ctypes.c_void_p * self.world)(*self.peer_ptrs)

    def ptr_array(self):
        return self._arr

    def mc(self):
        return ctypes.c_void_p(self.mc_ptr) if self.mc_ptr else ctypes.c_void_p(0)

    def peer_tensor(self, rank: int, shape, dtype, offset_elems: int = 0) -> torch.Tensor:
        return self.handle.get_buffer(rank, shape, dtype, offset_elems)


class SymmetricSlice:
    """A sub-range of a symmetric arena with the interface of ``SymmetricBuffer``: the arena was
    exchanged once, so the slice's peer and multicast addresses are the arena's plus the offset
    (the same on every rank, because every rank makes the same allocation calls)."""

    def __init__(self, arena: "SymmetricBuffer", offset: int, numel: int, dtype: torch.dtype, release=None):
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        self.arena, self.offset, self._release = arena, offset, release
        self.local = arena.local[offset:offset + nbytes].view(dtype)
        self.handle, self.world, self.rank = arena.handle, arena.world, arena.rank
        self.peer_ptrs = [p + offset for p in arena.peer_ptrs]
        self.mc_ptr = arena.mc_ptr + offset if arena.mc_ptr else 0
        self._arr = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        self._esz = nbytes // max(numel, 1)

    def ptr_array(self):
        return self._arr

    def mc(self):
        return ctypes.c_void_p(self.mc_ptr) if self.mc_ptr else ctypes.c_void_p(0)

    def peer_tensor(self, rank: int, shape, dtype, offset_elems: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        return self.handle.get_buffer(rank, shape, dtype, self.offset // esz + offset_elems)

    def free(self) -> None:
        """Returns the range to the arena (every rank must do so at the same point of its program)."""
        if self._release is not None:
            self._release(self.offset)
            self._release = None


class SymmetricHeap:
    """Allocator of symmetric buffers for one process group, plus the communicator state the
    fused kernels need: a zero-initialised signal array per rank and a call epoch.

    Two modes.  By default every ``allocate`` makes its own symmetric allocation and exchanges its
    handles (a rendezvous of all ranks).  With ``arena_bytes`` (or ``AXONML_SYMM_ARENA_MB``) the
    heap makes ONE symmetric allocation at construction and serves ``allocate`` from it through the
    native offset allocator (``csrc/host/arena.cpp``): no further rendezvous, one multicast binding
    for everything, and buffers can be given back (``SymmetricSlice.free``).  A request that does not
    fit falls back to an allocation of its own."""

    def __init__(self, pg, arena_bytes: int | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self.pg = pg
        grp = getattr(pg.backend(), "group", lambda: None)()
        self.group = grp if grp is not None else dist.group.WORLD
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.use_mc = os.environ.get("AXONML_NVLS", "1") != "0"
        self.rank, self.world = pg.rank(), pg.world_size()
        if arena_bytes is None:
            arena_bytes = int(os.environ.get("AXONML_SYMM_ARENA_MB", "0")) << 20
        self._arena = self._offsets = None
        if arena_bytes > 0:
            from ..core.storage import OffsetArena
            self._arena = self._allocate_own(arena_bytes, torch.uint8)
            self._offsets = OffsetArena(arena_bytes, 4096)

    def _allocate_own(self, numel: int, dtype: torch.dtype) -> SymmetricBuffer:
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        t.zero_()
        hdl = self._symm.rendezvous(t, self.group)
        return SymmetricBuffer(t, hdl, self.use_mc)

    def allocate(self, numel: int, dtype: torch.dtype):
        if self._offsets is not None:
            nbytes = numel * torch.empty((), dtype=dtype).element_size()
            off = self._offsets.alloc(nbytes)
            if off >= 0:
                sl = SymmetricSlice(self._arena, off, numel, dtype, release=self._offsets.free)
                sl.local.zero_()
                return sl
        return self._allocate_own(numel, dtype)

    def arena_stats(self) -> dict | None:
        return self._offsets.stats() if self._offsets is not None else None

    def barrier(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(self.group)


class Communicator:
    """Signal array + epoch counter + fixed grid for the kernels of ``csrc/kernels/comm.cu``."""

    def __init__(self, heap: SymmetricHeap, grid_blocks: int = 32):
        self.heap = heap
        slots = N.cuda().ax_comm_signal_slots()
        self.signals = heap.allocate(max(slots, 64), torch.int32)
        self.epoch = 0
        self.grid = grid_blocks
        heap.barrier()     # every rank's signal array is zero before anyone signals

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch
