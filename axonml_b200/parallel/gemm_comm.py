"""Driver of the fused tensor-parallel GEMM + collective kernels (``csrc/kernels/gemm_comm.cu``).

``FusedGemmComm.all_gather_linear``: all-gather of the token-sharded input fused into the GEMM of a
column-parallel layer.  ``FusedGemmComm.linear_reduce_scatter``: GEMM of a row-parallel layer whose
epilogue pushes finished tiles to the rank that owns those tokens, followed in the same launch by
the reduction of the local shard.  Both keep their peer-visible operands (gathered input, staging
slots, flags) in symmetric memory that is sized on first use and grown when a larger call arrives;
every rank makes the same calls in the same order, so the growth is collective.

Backward passes use the process group's collectives around the plain GEMM (Megatron style:
re-gather the input for the weight gradient), so the layers train; the forward is the fused path.

Reference semantics: ColumnParallelLinear / RowParallelLinear of
crates/axonml-distributed/src/fsdp.rs:414-600 (there: all_gather / all_reduce on a mock backend
around a CPU matmul).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as N
from ..ops.gemm import ACT, gemm_bf16
from ..ops import elementwise as E
from .symm import SymmetricHeap, available

_MAX_TILES = 4096
_PUSHER_GBS = 17.0        # bytes one copy CTA moves per second towards the peers (measured, GB/s)


def _pushers(tl: int, k: int, n: int, world: int, grid: int, multimem: bool) -> int:
    """Copy CTAs for the all-gather: enough that the shard is out before the GEMM has finished the
    local shard's tiles, no more (every copy CTA is one SM less for the math)."""
    local_gemm_s = 2.0 * tl * k * n / 1.4e15
    copies = 1 if (multimem and world > 2) else world - 1
    need = tl * k * 2 * copies / (_PUSHER_GBS * 1e9) / max(0.7 * local_gemm_s, 1e-6)
    return int(min(max(need + 0.999, 4), 24, grid // 4))


class _Channel:
    """One direction's symmetric state: data buffer, signal array, epoch."""

    def __init__(self, heap: SymmetricHeap):
        self.heap = heap
        slots = N.cuda().ax_gemm_comm_signal_slots(_MAX_TILES)
        self.sig = heap.allocate(slots, torch.int32)
        self.data = None
        self.capacity = 0
        self.epoch = 0
        heap.barrier()

    def ensure(self, numel: int) -> None:
        if numel > self.capacity:
            # all ranks reach this together; the old buffer is no longer written by any peer
            # because every earlier call has been consumed (the kernels' end-of-call signal)
            self.heap.barrier()
            self.data = self.heap.allocate(numel, torch.bfloat16)
            self.capacity = numel
            self.heap.barrier()


class FusedGemmComm:
    def __init__(self, pg):
        self.pg = pg
        self.heap = SymmetricHeap(pg)
        self.rank, self.world = self.heap.rank, self.heap.world
        self.ag = _Channel(self.heap)
        self.rs = _Channel(self.heap)
        self.grid = torch.cuda.get_device_properties(self.heap.device).multi_processor_count

    @classmethod
    def try_create(cls, pg):
        if not (available(pg) and N.is_blackwell()) or pg.world_size() > 8:
            return None
        return cls(pg)

    # ------------------------------------------------------------------ shape checks
    @staticmethod
    def _ok(x2, weight) -> bool:
        return (x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and x2.dim() == 2 and weight.dim() == 2 and x2.shape[1] == weight.shape[1]
                and x2.shape[1] % 64 == 0 and weight.shape[0] % 128 == 0)

    def supports_ag(self, x_local, weight) -> bool:
        return self._ok(x_local, weight) and x_local.shape[0] % 128 == 0 and x_local.shape[0] // 128 <= _MAX_TILES

    def supports_rs(self, x, weight) -> bool:
        if not self._ok(x, weight) or x.shape[0] % (128 * self.world):
            return False
        tl, n = x.shape[0] // self.world, weight.shape[0]
        bn = 256 if n % 256 == 0 else 128
        return (tl // 128) * (n // bn) <= _MAX_TILES

    # ------------------------------------------------------------------ raw launches
    def _launch(self, mode, ch, x, weight, out, bias, act, tl, n, k):
        ch.epoch += 1
        bias_kind = 0
        if bias is not None:
            bias = bias.contiguous()
            bias_kind = 1 if bias.dtype == torch.float32 else 2
        rc = N.cuda().ax_gemm_comm(
            mode, N.ptr(x), N.ptr(weight), N.ptr(out), ch.data.ptr_array(), ch.data.mc(), ch.sig.ptr_array(),
            N.ptr(bias), bias_kind, ACT[act], tl, n, k, self.rank, self.world, ctypes.c_uint(ch.epoch),
            _MAX_TILES, _pushers(tl, k, n, self.world, self.grid, bool(ch.data.mc_ptr)), self.grid,
            N.ptr(N.status_word(x.device)), N.stream_ptr())
        N.check(rc, "ax_gemm_comm")

    def ag_gemm(self, x_local, weight, bias=None, act="none"):
        x_local, weight = x_local.contiguous(), weight.contiguous()
        tl, k = x_local.shape
        n = weight.shape[0]
        self.ag.ensure(self.world * tl * k)
        out = torch.empty((self.world * tl, n), dtype=torch.bfloat16, device=x_local.device)
        self._launch(0, self.ag, x_local, weight, out, bias, act, tl, n, k)
        return out

    def gemm_rs(self, x, weight, bias=None, act="none"):
        x, weight = x.contiguous(), weight.contiguous()
        t, k = x.shape
        tl, n = t // self.world, weight.shape[0]
        self.rs.ensure(self.world * tl * n)
        out = torch.empty((tl, n), dtype=torch.bfloat16, device=x.device)
        self._launch(1, self.rs, x, weight, out, bias, act, tl, n, k)
        return out

    # ------------------------------------------------------------------ autograd entries
    def all_gather_linear(self, x_local, weight, bias=None, act="none"):
        if torch.is_grad_enabled() and (x_local.requires_grad or weight.requires_grad):
            y = _AGLinear.apply(x_local, weight, bias, self)
            if act not in ("none", None):
                from ..ops.linear import _ACT_FWD
                y = _ACT_FWD[act](y)        # differentiable torch op on the fused result
            return y
        return self.ag_gemm(x_local, weight, bias, act or "none")

    def linear_reduce_scatter(self, x, weight):
        if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
            return _LinearRS.apply(x, weight, self)
        return self.gemm_rs(x, weight)


def _all_gather_rows(t, eng):
    out = torch.empty((eng.world * t.shape[0], t.shape[1]), dtype=t.dtype, device=t.device)
    eng.pg.backend().all_gather(t.contiguous(), out.view(eng.world, t.shape[0], t.shape[1]))
    return out


def _reduce_scatter_rows(t, eng):
    from .backend import ReduceOp
    out = torch.empty((t.shape[0] // eng.world, t.shape[1]), dtype=t.dtype, device=t.device)
    eng.pg.backend().reduce_scatter(t.contiguous(), out, ReduceOp.Sum)
    return out


class _AGLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, bias, eng):
        ctx.eng = eng
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.save_for_backward(x_local, weight)
        return eng.ag_gemm(x_local, weight, bias, "none")

    @staticmethod
    def backward(ctx, dy):
        x_local, weight = ctx.saved_tensors
        eng = ctx.eng
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _reduce_scatter_rows(gemm_bf16(dy, weight, trans_b=False), eng)
        if ctx.needs_input_grad[1]:
            dw = gemm_bf16(dy, _all_gather_rows(x_local, eng), trans_a=True, trans_b=False)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = E.colsum(dy).to(ctx.bias_dtype)
        return dx, dw, db, None


class _LinearRS(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eng):
        ctx.eng = eng
        ctx.save_for_backward(x, weight)
        return eng.gemm_rs(x, weight)

    @staticmethod
    def backward(ctx, dy_local):
        x, weight = ctx.saved_tensors
        eng = ctx.eng
        dx = dw = None
        dy = _all_gather_rows(dy_local.contiguous(), eng)
        if ctx.needs_input_grad[0]:
            dx = gemm_bf16(dy, weight, trans_b=False)
        if ctx.needs_input_grad[1]:
            dw = gemm_bf16(dy, x, trans_a=True, trans_b=False)
        return dx, dw, None
