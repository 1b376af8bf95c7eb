"""Python drivers of the fused compute+collective kernels (``csrc/kernels/comm.cu``).

* ``FusedAllReduce``    - DDP bucket mean all-reduce + GradScaler unscale + found-inf, one kernel.
* ``FusedShardedAdamW`` - FSDP reduce-scatter + sharded AdamW, one kernel per flat unit; or, for LAMB,
  reduce-scatter + the first LAMB phase (moments, update, per-tensor sums of squares), the second
  phase following once the sums of all units have been added over the ranks.

Both keep their operands in symmetric memory: DDP allocates its gradient buckets inside the
all-reduce's symmetric arena, so a bucket is reduced in place (a tensor from elsewhere is staged
through the arena), FSDP allocates its flat gradient arena symmetrically.  The NCCL path
(``all_reduce`` / ``reduce_scatter_tensor``) remains the fallback and the baseline that the fused
path is measured against.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as N
from .symm import Communicator, SymmetricHeap, available


class FusedAllReduce:
    def __init__(self, heap: SymmetricHeap, max_numel: int, dtype: torch.dtype, grid_blocks: int = 32,
                 device_epoch: bool = False):
        """``device_epoch``: keep the call counter in device memory so that calls can be captured
        in CUDA graphs (serving decode steps); such an instance must not be mixed with host-counted
        calls."""
        self.heap = heap
        self.comm = Communicator(heap, grid_blocks)
        self.dtype = dtype
        self._epoch_dev = torch.zeros(1, dtype=torch.int32, device=heap.device) if device_epoch else None
        align = 8 * heap.world * 16
        self.capacity = (max_numel + align - 1) // align * align
        self.stage = heap.allocate(self.capacity, dtype)
        self._small = None
        if device_epoch:            # serving: the one-trip path for decode-sized vectors, allocated before any capture
            self._alloc_small()

    @classmethod
    def try_create(cls, pg, max_numel: int, dtype: torch.dtype, grid_blocks: int = 32, device_epoch: bool = False):
        if not available(pg) or dtype not in (torch.float32, torch.bfloat16):
            return None
        return cls(SymmetricHeap(pg), max_numel, dtype, grid_blocks, device_epoch)

    def holds(self, flat: torch.Tensor) -> bool:
        """True when ``flat`` can be reduced by this instance: it lies inside the symmetric arena
        (reduced in place) or fits into it (staged)."""
        return flat.dtype == self.dtype and flat.numel() <= self.capacity

    def all_reduce_mean_(self, flat: torch.Tensor, inv_scale=None, found_inf=None) -> None:
        """In-place mean over ranks of ``flat`` (optionally times ``inv_scale``); sets
        ``found_inf`` (int32[1]) when any reduced value is not finite.  A tensor that is a slice of
        this instance's symmetric arena (DDP allocates its buckets there) is reduced where it is;
        any other tensor is copied into the arena and back."""
        n = flat.numel()
        if n > self.capacity or flat.dtype != self.dtype:
            raise ValueError("bucket does not fit the fused all-reduce staging buffer")
        esz = flat.element_size()
        unit = 16 * self.heap.world // esz
        n_pad = (n + unit - 1) // unit * unit
        stage = self.stage.local
        off = flat.data_ptr() - stage.data_ptr()
        # in place only for a whole number of 16-byte-per-rank units: a ragged slice is staged instead
        in_place = (0 <= off and off + n * esz <= self.capacity * esz and off % 16 == 0 and n_pad == n
                    and flat.is_contiguous())
        if not in_place:
            off = 0
            stage[:n].copy_(flat)
            if n_pad > n:
                stage[n:n_pad].zero_()
        rc = N.cuda().ax_fused_allreduce(
            1 if self.dtype == torch.bfloat16 else 0, self.stage.ptr_array(),
            self.comm.signals.ptr_array(), self.stage.mc(), self.heap.rank, self.heap.world,
            ctypes.c_long(off), ctypes.c_long(n_pad), N.ptr(inv_scale), N.ptr(found_inf),
            ctypes.c_uint(0 if self._epoch_dev is not None else self.comm.next_epoch()), N.ptr(self._epoch_dev),
            self.comm.grid, N.ptr(N.status_word(flat.device)), N.stream_ptr())
        N.check(rc, "ax_fused_allreduce")
        if not in_place:
            flat.copy_(stage[:n])


    # ------------------------------------------------------------------ small vectors (decode)
    SMALL_BYTES = 64 * 1024

    def _alloc_small(self) -> None:
        self._small = self.heap.allocate(2 * self.heap.world * self.SMALL_BYTES // 2, torch.bfloat16)
        self._small_epoch = torch.zeros(1, dtype=torch.int32, device=self.heap.device)
        self.heap.barrier()

    def sum_small_(self, x: torch.Tensor, scale: float = 1.0) -> bool:
        """In-place ``x = scale * sum over ranks of x`` for a contiguous vector of at most
        ``SMALL_BYTES`` (a multiple of 16 bytes) through the one-trip kernel: every rank writes its
        vector into every rank's staging area and adds what it received.  ``x`` is an ordinary
        tensor (no staging copy).  Graph-capturable: the call counter is on the device.  Returns
        False (nothing done) when the vector does not qualify."""
        nbytes = x.numel() * x.element_size()
        if (x.dtype != self.dtype or not x.is_contiguous() or nbytes > self.SMALL_BYTES or nbytes % 16
                or x.data_ptr() % 16):
            return False
        if self._small is None:
            self._alloc_small()
        rc = N.cuda().ax_oneshot_allreduce(
            1 if self.dtype == torch.bfloat16 else 0, self._small.ptr_array(), self.comm.signals.ptr_array(),
            self._small.mc(), self.heap.rank, self.heap.world, N.ptr(x), N.ptr(x), ctypes.c_long(nbytes),
            ctypes.c_long(self.SMALL_BYTES), ctypes.c_float(scale), N.ptr(self._small_epoch),
            N.ptr(N.status_word(x.device)), N.stream_ptr())
        N.check(rc, "ax_oneshot_allreduce")
        return True


class FusedShardedAdamW:
    """Owns the symmetric gradient arena of a sharded engine and steps one unit per call."""

    def __init__(self, heap: SymmetricHeap, arena_numel: int, grid_blocks: int = 32):
        self.heap = heap
        self.comm = Communicator(heap, grid_blocks)
        self.arena = heap.allocate(arena_numel, torch.bfloat16)

    def step_unit(self, grad_off_elems: int, shard: int, master, m1, m2, lp, *, lr, beta1, beta2, eps,
                  wd, step: int, skip_flag=None) -> None:
        hyper = (ctypes.c_float * 7)(lr, beta1, beta2, eps, wd, 1 - beta1 ** step, 1 - beta2 ** step)
        rc = N.cuda().ax_fused_rs_adamw(
            self.arena.ptr_array(), self.comm.signals.ptr_array(), self.arena.mc(), self.heap.rank,
            self.heap.world, ctypes.c_long(grad_off_elems * 2), ctypes.c_long(shard), N.ptr(master),
            N.ptr(m1), N.ptr(m2), N.ptr(lp), hyper, N.ptr(skip_flag),
            ctypes.c_uint(self.comm.next_epoch()), self.comm.grid, N.ptr(N.status_word(master.device)),
            N.stream_ptr())
        N.check(rc, "ax_fused_rs_adamw")

    def step_unit_lamb1(self, grad_off_elems: int, shard: int, master, m1, m2, upd, seg_start, seg_gid, norms, *,
                        beta1, beta2, eps, wd, step: int, bias_correction: bool = True, skip_flag=None) -> None:
        """Reduce-scatter of one unit's flat gradient fused with the first LAMB phase (moments, the
        per-element update into ``upd``, this shard's share of the per-tensor sums of squares into
        ``norms``)."""
        bc1 = 1 - beta1 ** step if bias_correction else 1.0
        bc2 = 1 - beta2 ** step if bias_correction else 1.0
        hyper = (ctypes.c_float * 7)(0.0, beta1, beta2, eps, wd, bc1, bc2)
        rc = N.cuda().ax_fused_rs_lamb1(
            self.arena.ptr_array(), self.comm.signals.ptr_array(), self.arena.mc(), self.heap.rank, self.heap.world,
            ctypes.c_long(grad_off_elems * 2), ctypes.c_long(shard), N.ptr(master), N.ptr(m1), N.ptr(m2), N.ptr(upd),
            N.ptr(seg_start), N.ptr(seg_gid), int(seg_gid.numel()), N.ptr(norms), hyper, N.ptr(skip_flag),
            ctypes.c_uint(self.comm.next_epoch()), self.comm.grid, N.ptr(N.status_word(master.device)), N.stream_ptr())
        N.check(rc, "ax_fused_rs_lamb1")
