"""Driver of the fused tensor-parallel GEMM + collective kernels (``csrc/kernels/gemm_comm.cu``).

``FusedGemmComm.all_gather_linear``: all-gather of the token-sharded input fused into the GEMM of a
column-parallel layer.  ``FusedGemmComm.linear_reduce_scatter``: GEMM of a row-parallel layer whose
epilogue pushes finished tiles to the rank that owns those tokens, followed in the same launch by
the reduction of the local shard.  Both keep their peer-visible operands (gathered input, staging
slots, flags) in symmetric memory that is sized on first use and grown when a larger call arrives;
every rank makes the same calls in the same order, so the growth is collective.

Backward passes run on the same kernels.  The input gradient of a column-parallel layer is a
GEMM -> reduce-scatter with the weight read as ``[K, N]``; its weight gradient reads the gathered
input that the forward launch left, complete, in a symmetric buffer kept for that layer (no second
all-gather; the buffers are kept while they fit ``AXONML_TP_KEEP_GB``, 48 GB by default, and a
layer without one re-gathers through the process group).  The input gradient of a row-parallel
layer is an all-gather -> GEMM of the output gradient, whose gathered copy then feeds the weight
gradient.

Reference semantics: ColumnParallelLinear / RowParallelLinear of
crates/axonml-distributed/src/fsdp.rs:414-600 (there: all_gather / all_reduce on a mock backend
around a CPU matmul).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from .. import _native as N
from ..ops.gemm import ACT, gemm_bf16
from ..ops import elementwise as E
from .symm import SymmetricHeap, available

_MAX_TILES = 4096
_PUSHER_GBS = 22.0        # what one copy CTA sends per second (700 GB/s from 32 CTAs, measured)
_PUSHER_MC_GBS = 11.0     # the same through multimem stores (4 GPUs: 8 copy CTAs deliver a 33.5 MB shard in 365 us)
_LINK_GBS = 700.0         # what a GPU receives per second over NVLink (measured peer copy)


def _pushers(tl: int, k: int, n: int, world: int, grid: int, multimem: bool) -> int:
    """Copy CTAs for the all-gather: enough to send this rank's shard within the time the launch
    has anyway (most of the GEMM, or the time the GPU needs to receive the other shards, whichever
    is longer), no more: every copy CTA is one SM less for the math.  With NVSwitch multicast a
    shard leaves the GPU once, whatever the number of peers."""
    forced = os.environ.get("AXONML_TP_PUSHERS")
    if forced:
        return int(min(max(int(forced), 1), grid // 2))
    gemm_s = 2.0 * world * tl * k * n / 1.4e15
    recv_s = (world - 1) * tl * k * 2 / (_LINK_GBS * 1e9)
    mc = multimem and world > 2
    copies = 1 if mc else world - 1
    rate = _PUSHER_MC_GBS if mc else _PUSHER_GBS
    need = tl * k * 2 * copies / (rate * 1e9) / max(0.6 * gemm_s, recv_s, 1e-6)
    need = min(max(need, 2.0), 24.0, grid // 4)
    # a copy CTA takes whole 128-row chunks: with a count that does not divide the chunks some CTAs
    # run one round more than the others, which costs SMs without shortening the transfer
    chunks = max(tl // 128, 1)
    rounds = max(1, math.ceil(chunks / need - 1e-9))
    return int(max(2, min(math.ceil(chunks / rounds), grid // 4)))


class _Channel:
    """One direction's symmetric state: data buffer, signal array, epoch."""

    def __init__(self, heap: SymmetricHeap, keep: bool = False):
        self.heap = heap
        slots = N.cuda().ax_gemm_comm_signal_slots(_MAX_TILES)
        self.sig = heap.allocate(slots, torch.int32)
        self.data = None
        self.capacity = 0
        self.epoch = 0
        self.keep = keep          # gathered rows stay readable after the launch (see ax_gemm_comm)
        heap.barrier()

    def ensure(self, numel: int) -> None:
        if numel > self.capacity:
            # all ranks reach this together; the old buffer is no longer written by any peer
            # because every earlier call has been consumed (the kernels' end-of-call signal)
            self.heap.barrier()
            self.data = self.heap.allocate(numel, torch.bfloat16)
            self.capacity = numel
            self.heap.barrier()

    def gathered(self, rows: int, k: int) -> torch.Tensor:
        """This rank's copy of the rows gathered by the last call, ``[rows, k]``."""
        return self.data.local[:rows * k].view(rows, k)


class FusedGemmComm:
    def __init__(self, pg):
        self.pg = pg
        self.heap = SymmetricHeap(pg)
        self.rank, self.world = self.heap.rank, self.heap.world
        self.ag = _Channel(self.heap)
        self.rs = _Channel(self.heap)
        self.ag_bwd = _Channel(self.heap, keep=True)      # gathered output gradients of row-parallel layers
        self._kept: dict = {}                              # id(weight) -> channel holding that layer's gathered input
        self._kept_bytes = 0
        self._keep_budget = int(float(os.environ.get("AXONML_TP_KEEP_GB", "48")) * (1 << 30))
        self.grid = torch.cuda.get_device_properties(self.heap.device).multi_processor_count

    def kept_channel(self, weight, numel: int):
        """Symmetric buffer that keeps the gathered input of the layer owning ``weight`` between its
        forward and backward, or None when the budget is used up.  Every rank asks in the same
        order with the same sizes, so the allocation is collective."""
        ch = self._kept.get(id(weight))
        if ch is None:
            if self._kept_bytes + numel * 2 > self._keep_budget:
                return None
            ch = self._kept[id(weight)] = _Channel(self.heap, keep=True)
            ch.version = 0
        if numel > ch.capacity:
            if self._kept_bytes + (numel - ch.capacity) * 2 > self._keep_budget:
                return None
            self._kept_bytes += (numel - ch.capacity) * 2
        return ch

    @classmethod
    def try_create(cls, pg):
        if not (available(pg) and N.is_blackwell()) or pg.world_size() > 8:
            return None
        # AXONML_TP_RS=push|pull overrides the reduce-scatter transport (default: in-switch reduction
        # above two ranks when the buffers have a multicast mapping)
        mode = os.environ.get("AXONML_TP_RS", "auto")
        N.cuda().ax_gemm_comm_set_rs_pull({"push": 0, "pull": 1}.get(mode, -1))
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
    def _launch(self, mode, ch, x, weight, out, bias, act, tl, n, k, trans_b=True):
        ch.epoch += 1
        bias_kind = 0
        if bias is not None:
            bias = bias.contiguous()
            bias_kind = 1 if bias.dtype == torch.float32 else 2
        rc = N.cuda().ax_gemm_comm(
            mode, N.ptr(x), N.ptr(weight), N.ptr(out), ch.data.ptr_array(), ch.data.mc(), ch.sig.ptr_array(),
            N.ptr(bias), bias_kind, ACT[act], tl, n, k, int(not trans_b), self.rank, self.world,
            ctypes.c_uint(ch.epoch), _MAX_TILES, _pushers(tl, k, n, self.world, self.grid, bool(ch.data.mc_ptr)),
            self.grid, int(ch.keep), N.ptr(N.status_word(x.device)), N.stream_ptr())
        N.check(rc, "ax_gemm_comm")

    def ag_gemm(self, x_local, weight, bias=None, act="none", *, trans_b: bool = True, channel=None):
        """``act(all_gather(x_local) @ op(weight) + bias)``; ``trans_b=True``: weight is ``[N, K]``
        (a Linear weight), ``False``: weight is ``[K, N]``."""
        x_local, weight = x_local.contiguous(), weight.contiguous()
        tl, k = x_local.shape
        n = weight.shape[0] if trans_b else weight.shape[1]
        ch = channel or self.ag
        ch.ensure(self.world * tl * k)
        out = torch.empty((self.world * tl, n), dtype=torch.bfloat16, device=x_local.device)
        self._launch(0, ch, x_local, weight, out, bias, act, tl, n, k, trans_b)
        return out

    def gemm_rs(self, x, weight, bias=None, act="none", *, trans_b: bool = True):
        """This rank's rows of ``act(sum over ranks of x @ op(weight) + bias)``."""
        x, weight = x.contiguous(), weight.contiguous()
        t, k = x.shape
        n = weight.shape[0] if trans_b else weight.shape[1]
        tl = t // self.world
        self.rs.ensure(self.world * tl * n)
        out = torch.empty((tl, n), dtype=torch.bfloat16, device=x.device)
        self._launch(1, self.rs, x, weight, out, bias, act, tl, n, k, trans_b)
        return out

    def supports_bwd(self, rows_local: int, k: int, n: int) -> bool:
        """Shapes of the two backward launches of a layer with a ``[n, k]`` weight."""
        return k % 128 == 0 and n % 64 == 0 and rows_local % 128 == 0

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
        tl, k = x_local.shape
        ch = eng.kept_channel(weight, eng.world * tl * k)
        ctx.ch, ctx.version = ch, None
        if ch is not None:
            ch.version += 1
            ctx.version = ch.version
        return eng.ag_gemm(x_local, weight, bias, "none", channel=ch)

    @staticmethod
    def backward(ctx, dy):
        x_local, weight = ctx.saved_tensors
        eng = ctx.eng
        dy = dy.contiguous()
        dx = dw = db = None
        n, k = weight.shape
        fused = _fused_backward() and eng.supports_bwd(x_local.shape[0], k, n)
        if ctx.needs_input_grad[0]:
            if fused and k % 64 == 0 and n % 64 == 0:
                dx = eng.gemm_rs(dy, weight, trans_b=False)          # dy [T, n] @ weight [n, k] -> rows of this rank
            else:
                dx = _reduce_scatter_rows(gemm_bf16(dy, weight, trans_b=False), eng)
        if ctx.needs_input_grad[1]:
            ch = ctx.ch
            if ch is not None and ch.version == ctx.version:
                # the forward (or its recomputation) left the gathered input in this layer's buffer
                xg = ch.gathered(eng.world * x_local.shape[0], k)
            else:
                xg = _all_gather_rows(x_local, eng)
            dw = gemm_bf16(dy, xg, trans_a=True, trans_b=False)
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
        dy_local = dy_local.contiguous()
        n, k = weight.shape
        tl = dy_local.shape[0]
        if _fused_backward() and ctx.needs_input_grad[0] and tl % 128 == 0 and n % 64 == 0 and k % 128 == 0 \
                and tl // 128 <= _MAX_TILES:
            # all-gather of dy fused into dx = dy @ weight; the gathered dy stays for the weight gradient
            dx = eng.ag_gemm(dy_local, weight, trans_b=False, channel=eng.ag_bwd)
            if ctx.needs_input_grad[1]:
                dw = gemm_bf16(eng.ag_bwd.gathered(eng.world * tl, n), x, trans_a=True, trans_b=False)
            return dx, dw, None
        dy = _all_gather_rows(dy_local, eng)
        if ctx.needs_input_grad[0]:
            dx = gemm_bf16(dy, weight, trans_b=False)
        if ctx.needs_input_grad[1]:
            dw = gemm_bf16(dy, x, trans_a=True, trans_b=False)
        return dx, dw, None


def _fused_backward() -> bool:
    """``AXONML_TP_BWD=nccl`` composes the backward passes from process-group collectives and the
    plain GEMM (the baseline the fused backward is measured against)."""
    return os.environ.get("AXONML_TP_BWD", "fused") != "nccl"
