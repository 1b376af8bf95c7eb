"""FullyShardedDataParallel: ZeRO-2 / ZeRO-3 over flat-parameter units.

API of the reference (crates/axonml-distributed/src/fsdp.rs:33-354): ``ShardingStrategy``
{FullShard (ZeRO-3, default), ShardGradOp (ZeRO-2), NoShard, HybridShard}, ``CPUOffload``,
builders ``sharding_strategy / cpu_offload / mixed_precision``, ``gather_parameters``,
``reshard_parameters``, ``sync_gradients``, ``clip_grad_norm``, ``memory_estimate``; alias
``FSDP``.  The reference shards every parameter separately, never gathers in ``forward`` and drops
the result of its reduce-scatter (fsdp.rs:259-268, :350-354); here the engine is real:

* one flat unit per transformer block (plus a root unit for what is left), see ``flat_param``;
* forward / recompute / backward gather a unit's parameters just in time on a communication
  stream and prefetch the next unit while the current one computes; with ``gather="fused"`` (B200s
  with symmetric memory, bf16, more than one rank) the forward and the recomputed forward do not
  gather at all: the first Linear of a unit runs as ONE kernel that gathers the unit's flat buffer
  over peer memory and computes that Linear, its weight loads gated on the arrival of the rows they
  read (``csrc/kernels/gemm_gather.cu``).  For this the 1-D parameters of the units (norm weights,
  biases) move into the root unit, which is gathered once per step, so that everything a unit
  gathers is first touched by a GEMM.  ``gather="auto"`` takes the prefetching NCCL gathers: on the
  GPT-1.3B step they hide completely behind the previous unit's compute (116.7 ms/step on 8 GPUs
  against 119.7 ms with the fused gather, whose copy CTAs take SMs from the GEMM they feed and whose
  transfer cannot start before that GEMM does), so the fused form only pays where there is no
  earlier compute to hide a gather behind;
* ZeRO-3 with more than one rank rotates three full-size buffers between the block units (a
  unit's parameters always view the same buffer, so no pointer is ever re-bound); ZeRO-2, NoShard
  and single-rank runs keep one resident buffer per unit;
* when the last gradient of a unit has arrived its flat gradient is reduce-scattered (mean) on the
  communication stream while backward continues;
* the optimizer steps fp32 master shards (``parameters()``), and its fused kernel writes the bf16
  shard in the same pass.
"""
from __future__ import annotations

import contextlib
import dataclasses
import enum
import os

import torch
import torch.distributed as dist

from ..nn.module import Module
from .backend import ReduceOp
from .flat_param import FlatUnit
from .process_group import ProcessGroup


class ShardingStrategy(enum.Enum):
    FullShard = "full_shard"        # ZeRO-3
    ShardGradOp = "shard_grad_op"   # ZeRO-2
    NoShard = "no_shard"            # DDP-like
    HybridShard = "hybrid_shard"    # shard inside a node, replicate across (single node: = FullShard)


class CPUOffload(enum.Enum):
    None_ = "none"
    Params = "params"
    Full = "full"


@dataclasses.dataclass
class FSDPMemoryStats:
    total_params: int
    total_param_memory: int
    local_params: int
    local_param_memory: int
    local_optimizer_memory: int
    savings_factor: float
    world_size: int = 1

    def total_memory_mb(self) -> float:
        """Parameters (with their fp32 masters) plus optimizer state held by this rank, in MiB."""
        return (self.local_param_memory + self.local_optimizer_memory) / (1024.0 * 1024.0)

    def memory_savings(self) -> float:
        """Fraction of the unsharded footprint this rank no longer holds: 1 - 1 / world size."""
        return 1.0 - 1.0 / self.world_size if self.world_size > 1 else 0.0


class _Buffer:
    def __init__(self, numel, dtype, device, heap=None):
        self.sym = self.sig = None
        self.epoch = 0
        if heap is not None:
            # symmetric memory: peers write their shards into this buffer from inside the fused
            # gather + GEMM kernel; `sig` holds that kernel's flags
            from .. import _native as N
            self.sym = heap.allocate(numel, dtype)
            self.data = self.sym.local
            self.sig = heap.allocate(max(int(N.cuda().ax_gemm_gather_signal_slots(numel, heap.world)), 64), torch.int32)
            heap.barrier()
        else:
            self.data = torch.zeros(numel, dtype=dtype, device=device)
        self.owner = None
        self.free_event = None


class _GatherGate:
    """Pending gather of one unit, carried by the unit's 2-D weights (``_axon_gate``): the first
    Linear that runs on one of them turns it into the fused gather + GEMM launch."""

    def __init__(self, engine, unit):
        self.engine, self.unit = engine, unit
        self.pending = False
        self.linear_only = True      # every 2-D weight of the unit belongs to a Linear (which checks the gate)

    def usable(self, x2, w, act_needs_aux: bool) -> bool:
        return (self.pending and not act_needs_aux and x2.dtype == torch.bfloat16
                and w.shape[1] % 64 == 0 and w.shape[0] % 8 == 0 and x2.shape[0] > 0)

    def gemm(self, x2, w, bias, act: str):
        """``act(x2 @ w.T + bias)`` with the gather of the whole unit inside the same launch."""
        import ctypes
        from .. import _native as N
        from ..ops.gemm import ACT
        u, eng = self.unit, self.engine
        buf = u.buffer
        buf.epoch += 1
        w_off = (w.data_ptr() - u.full.data_ptr()) // 2
        out = torch.empty((x2.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x2.device)
        bias_kind = 0
        if bias is not None:
            bias = bias.contiguous()
            bias_kind = 1 if bias.dtype == torch.float32 else 2
        # what one copy CTA moves per second (measured on peer copies); the gather has the time of
        # the GEMM to finish, a multicast store leaves the GPU once
        copies = 1 if (buf.sym.mc_ptr and eng.world > 2) else eng.world
        gemm_s = 2.0 * x2.shape[0] * w.shape[0] * w.shape[1] / 1.4e15
        need = u.shard * 2 * copies / 22e9 / max(0.5 * gemm_s, 2e-5)
        copy_pairs = int(min(max(need / 2 + 0.999, 1), 12))
        rc = N.cuda().ax_gemm_gather(
            N.ptr(x2), N.ptr(out), N.ptr(bias), bias_kind, ACT[act], x2.shape[0], w.shape[0], w.shape[1],
            ctypes.c_long(w_off), ctypes.c_long(u.padded), N.ptr(u.lp_shard), buf.sym.ptr_array(), buf.sym.mc(),
            buf.sig.ptr_array(), eng.rank, eng.world, ctypes.c_uint(buf.epoch), copy_pairs,
            N.ptr(N.status_word(x2.device)), N.stream_ptr())
        N.check(rc, "ax_gemm_gather")
        self.pending = False
        eng._mark_gathered(u)
        eng.fused_gathers += 1
        return out

    def fallback(self) -> None:
        """The first consumer is not a Linear this kernel can take: gather the plain way, now."""
        self.pending = False
        self.engine._gather(self.unit)
        self.engine._wait(self.unit)


class FullyShardedDataParallel(Module):
    def __init__(self, module: torch.nn.Module, process_group: ProcessGroup | None = None, *,
                 units: list | None = None, param_dtype: torch.dtype | None = None,
                 strategy: ShardingStrategy = ShardingStrategy.FullShard, device=None,
                 fused_adamw: dict | None = None, fused_lamb: dict | None = None, gather: str = "auto"):
        super().__init__()
        self.module = module
        self.pg = process_group or ProcessGroup.mock()
        self.world, self.rank = self.pg.world_size(), self.pg.rank()
        self._strategy = strategy
        self._cpu_offload = CPUOffload.None_
        self._mixed_precision = True
        first = next(module.parameters())
        self.device = torch.device(device) if device is not None else first.device
        self.param_dtype = param_dtype or first.dtype
        self._group = getattr(self.pg.backend(), "group", lambda: None)()
        self._use_dist = self.world > 1 and dist.is_initialized()
        self._unit_modules = units
        self._built = False
        self._phase = "idle"
        self._sync = True
        if fused_adamw and fused_lamb:
            raise ValueError("give fused_adamw or fused_lamb, not both")
        self._fused_hp = dict(fused_adamw or fused_lamb) if (fused_adamw or fused_lamb) else None
        self._fused_kind = "lamb" if fused_lamb else "adamw"
        self._fused = None
        self._fused_step = 0
        self._fused_pending = False
        self._gather_mode = os.environ.get("AXONML_FSDP_GATHER", gather)
        self._k4 = False
        self.fused_gathers = 0           # launches of the fused gather + GEMM kernel so far
        self._build()

    # ------------------------------------------------------------------ reference builders
    @classmethod
    def new(cls, module, process_group): return cls(module, process_group)

    def sharding_strategy(self, strategy: ShardingStrategy):
        if strategy is not self._strategy:
            raise ValueError("pass strategy= at construction; units are laid out for one strategy")
        return self

    def cpu_offload(self, offload: CPUOffload):
        """``Params`` / ``Full`` (fsdp.rs:70-83): the fp32 master shards, and with them the optimizer
        state that is created from them, live in pinned host memory; the optimizer steps there and
        the low-precision shard on the device is refreshed from the host after each step.  The
        reduced gradient shard is copied to the host at the end of backward (``Full`` also drops
        the device copy's role: accumulation over backward calls happens on the host).  Call this
        before the optimizer is created.  Not available with the in-backward fused AdamW, whose
        state is on the device by construction."""
        if offload is not CPUOffload.None_ and self._fused is not None:
            raise ValueError("cpu_offload cannot be combined with fused_adamw (its master weights and moments "
                             "are updated on the device inside backward)")
        if offload is self._cpu_offload:
            return self
        self._cpu_offload = offload
        to_host = offload is not CPUOffload.None_
        for u in self.units:
            grad, lp = u.master._axon_grad, u.master._axon_lp
            with torch.no_grad():
                if to_host:
                    host = u.master.data.detach().to("cpu")
                    if torch.cuda.is_available():
                        host = host.pin_memory()
                    u.master.data = host
                    u.grad_host = torch.zeros(u.shard, dtype=self.param_dtype, device="cpu")
                    if torch.cuda.is_available():
                        u.grad_host = u.grad_host.pin_memory()
                else:
                    u.master.data = u.master.data.to(self.device)
                    u.grad_host = None
            u.master._axon_lp = lp
            u.master._axon_grad = None if to_host else grad
        return self

    def mixed_precision(self, flag: bool):
        """The engine computes in ``param_dtype`` and steps fp32 master shards.  ``False`` asks for
        full-precision compute, which is what ``param_dtype=torch.float32`` at construction gives;
        the parameter buffers are laid out for one dtype, so it cannot be switched afterwards."""
        if not flag and self.param_dtype != torch.float32:
            raise ValueError("pass param_dtype=torch.float32 at construction for full-precision compute")
        self._mixed_precision = flag
        return self

    def strategy(self) -> ShardingStrategy: return self._strategy

    # ------------------------------------------------------------------ construction
    def _auto_units(self):
        mods = []
        for m in self.module.modules():
            if isinstance(m, torch.nn.ModuleList) and len(m) > 1 and all(
                    any(True for _ in c.parameters()) for c in m):
                mods.extend(list(m))
        return mods

    def _build(self):
        unit_mods = self._unit_modules if self._unit_modules is not None else self._auto_units()
        seen = set()
        self.units: list[FlatUnit] = []
        self._unit_of_module = {}
        shard_params = self._strategy is not ShardingStrategy.NoShard
        w = self.world if shard_params else 1
        r = self.rank if shard_params else 0
        self._k4 = self._want_fused_gather(unit_mods)
        for i, m in enumerate(unit_mods):
            ps = [p for p in m.parameters() if id(p) not in seen and p.requires_grad
                  and (p.dim() >= 2 or not self._k4)]     # fused gather: 1-D parameters go to the root unit
            for p in ps:
                seen.add(id(p))
            if not ps:
                continue
            u = FlatUnit(f"unit{i}", ps, w, r, self.device, self.param_dtype)
            u.module, u.is_root, u.index = m, False, len(self.units)
            self.units.append(u)
            self._unit_of_module[id(m)] = u
        rest = [p for p in self.module.parameters() if id(p) not in seen and p.requires_grad]
        self.root = None
        if rest:
            u = FlatUnit("root", rest, w, r, self.device, self.param_dtype)
            u.module, u.is_root, u.index = self.module, True, -1
            self.root = u
        self.block_units = list(self.units)
        if self.root is not None:
            self.units.append(self.root)

        rotate = (self._strategy in (ShardingStrategy.FullShard, ShardingStrategy.HybridShard)
                  and self.world > 1 and len(self.block_units) > 3)
        self._rotate = rotate
        heap = None
        if self._k4:
            from .symm import SymmetricHeap
            heap = SymmetricHeap(self.pg)
        if rotate:
            size = max(u.padded for u in self.block_units)
            self._pool = [_Buffer(size, self.param_dtype, self.device, heap) for _ in range(3)]
        for u in self.units:
            if rotate and not u.is_root:
                u.buffer = self._pool[u.index % 3]
            else:
                u.buffer = _Buffer(u.padded, self.param_dtype, self.device, heap if (not u.is_root and u.world > 1) else None)
                u.buffer.owner = u
            u.bind_full(u.buffer.data[:u.padded])
            if u.world == 1:
                # the shard is the whole buffer: the optimizer writes the parameters directly
                u.full.copy_(u._init_full)
                u._init_full = None
                u.lp_shard = u.full
                u.gathered = True
            u.bind_grad(self._grad_storage(u))
            u.grad_shard = u.grad_flat if u.world == 1 else torch.zeros(
                u.shard, dtype=self.param_dtype, device=self.device)
            u.master._axon_lp = u.lp_shard
            u.master._axon_grad = None
        self._attach_segments()
        self._comm = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        if self._k4:
            from ..nn.layers.linear import Linear as _Linear
            for u in self.block_units:
                u.gate = _GatherGate(self, u)
                for p in u.params:
                    if p.dim() == 2:
                        p._axon_gate = u.gate
                # Safety net: a submodule that owns weights but does not go through ops.linear (which
                # consumes the gate) must find its weights gathered when its forward starts.
                own = {id(p) for p in u.params}
                for sub in u.module.modules():
                    if isinstance(sub, _Linear) or not any(id(p) in own for p in sub.parameters(recurse=False)):
                        continue
                    u.gate.linear_only = False
                    sub.register_forward_pre_hook(lambda m, a, g=u.gate: g.fallback() if g.pending else None)

        for u in self.block_units:
            u.module.register_forward_pre_hook(lambda m, a, u=u: self._pre_forward(u))
            u.module.register_forward_hook(lambda m, a, o, u=u: self._post_forward(u))
            u.module.register_full_backward_pre_hook(lambda m, g, u=u: self._pre_backward(u))
        for u in self.units:
            for idx, p in enumerate(u.params):
                p.register_post_accumulate_grad_hook(lambda p, u=u, idx=idx: self._on_grad(u, idx, p))
                if not u.is_root and p.dim() == 2:
                    p._axon_grad_sink = _GradSink(self, u, idx)
        self._built = True

    def _want_fused_gather(self, unit_mods) -> bool:
        """Whether the forward gathers of the block units run inside their first GEMM."""
        if self._gather_mode != "fused" or not unit_mods:
            return False
        ok = (self.world > 1 and self.device.type == "cuda" and self.param_dtype == torch.bfloat16
              and self._strategy in (ShardingStrategy.FullShard, ShardingStrategy.HybridShard))
        if ok:
            from .. import _native as N
            from .symm import available
            ok = available(self.pg) and N.is_blackwell() and self.world <= 8
        if not ok and self._gather_mode == "fused":
            raise ValueError("gather='fused' needs more than one rank on B200s with symmetric memory, bf16 parameters "
                             "and the FullShard strategy")
        return ok

    def _mark_gathered(self, u: FlatUnit) -> None:
        buf = u.buffer
        if buf.owner is not None and buf.owner is not u:
            buf.owner.gathered = False
        buf.owner = u
        u.gathered = True
        u.gather_event = None

    def _attach_segments(self) -> None:
        """Tells per-tensor optimizers (LAMB's trust ratio) which tensors a master shard holds:
        ``_axon_segments`` = [(tensor id over all units, start in the shard, length)] and a
        reduction that sums per-tensor statistics over the ranks holding the other slices."""
        gid = 0
        total = sum(len(u.params) for u in self.units)
        for u in self.units:
            lo, hi = u.rank * u.shard, (u.rank + 1) * u.shard
            segs = []
            for p, o in zip(u.params, u.offsets):
                a, b = max(o, lo), min(o + p.numel(), hi)
                segs.append((gid, a - lo, max(b - a, 0)))
                gid += 1
            u.master._axon_segments = segs
            u.master._axon_num_tensors = total
            if u.world > 1:
                u.master._axon_norm_reduce = lambda t: self.pg.backend().all_reduce(t, ReduceOp.Sum)

    def _grad_storage(self, u: FlatUnit) -> torch.Tensor:
        """Flat gradient of a unit: a slice of the symmetric arena when the fused reduce-scatter +
        AdamW kernel is in use, an ordinary tensor otherwise."""
        if self._fused_hp is not None and self._fused is None and self.world > 1 and u.world > 1:
            from . import fused as F
            from .symm import SymmetricHeap, available
            if available(self.pg) and self.param_dtype == torch.bfloat16:
                total = sum(x.padded for x in self.units)
                self._fused = F.FusedShardedAdamW(SymmetricHeap(self.pg), total)
                self._arena_off = 0
                for x in self.units:
                    x.m1 = torch.zeros(x.shard, dtype=torch.float32, device=self.device)
                    x.m2 = torch.zeros(x.shard, dtype=torch.float32, device=self.device)
                    if self._fused_kind == "lamb":
                        x.upd = torch.zeros(x.shard, dtype=torch.float32, device=self.device)
            else:
                self._fused_hp = None
        if self._fused is not None:
            u.grad_off = self._arena_off
            self._arena_off += u.padded
            return self._fused.arena.local[u.grad_off:u.grad_off + u.padded]
        return torch.zeros(u.padded, dtype=self.param_dtype, device=self.device)

    def _lamb_tables(self, u: FlatUnit) -> None:
        """Device tables for the fused LAMB kernel: where each tensor's slice starts inside this
        rank's shard of the unit and which tensor it is; one [tensors, 2] accumulator for all units."""
        if getattr(u, "seg_gid", None) is not None:
            return
        segs = [(gid, s, n) for gid, s, n in u.master._axon_segments if n > 0]
        starts = [s for _, s, _ in segs] + [u.shard]
        u.seg_start = torch.tensor(starts if segs else [0], dtype=torch.int64, device=self.device)
        u.seg_gid = torch.tensor([g for g, _, _ in segs], dtype=torch.int32, device=self.device)
        u.seg_list = segs
        if getattr(self, "_lamb_norms", None) is None:
            self._lamb_norms = torch.zeros(u.master._axon_num_tensors, 2, dtype=torch.float32, device=self.device)

    def _lamb_phase2(self) -> None:
        """Trust ratio per tensor from the sums of squares added over the ranks, then the update."""
        from ..ops import optim as O
        hp = self._fused_hp
        if getattr(self, "_lamb_norms", None) is None:
            return
        norms = self._lamb_norms
        if self.world > 1:
            self.pg.backend().all_reduce(norms, ReduceOp.Sum)
        ps, us, lps, gids = [], [], [], []
        for u in self.units:
            if getattr(u, "seg_list", None) is None or u.world == 1:
                continue
            w, lp = u.master.data, u.lp_shard
            for gid, s0, n in u.seg_list:
                ps.append(w[s0:s0 + n]); us.append(u.upd[s0:s0 + n]); lps.append(lp[s0:s0 + n]); gids.append(gid)
        if ps:
            rows = norms[torch.tensor(gids, dtype=torch.long, device=self.device)].contiguous()
            O.multi_tensor("lamb2", ps, us, us, us, us, lp=lps, lr=hp["lr"], norms=rows)
        norms.zero_()

    def fused_optimizer(self):
        """Handle with the optimizer API for the in-backward fused optimizer.  AdamW: ``step`` only
        advances the step counter, the update itself runs inside backward, fused with the
        reduce-scatter.  LAMB: backward runs the first phase inside the reduce-scatter kernel, ``step``
        adds the per-tensor sums over the ranks and applies the trust-ratio update."""
        return _FusedOptimizerHandle(self)

    # ------------------------------------------------------------------ gather / release
    def _stream_ctx(self):
        return torch.cuda.stream(self._comm) if self._comm is not None else contextlib.nullcontext()

    def _gather(self, u: FlatUnit) -> None:
        if u.gathered or u.world == 1:
            return
        buf = u.buffer
        with self._stream_ctx():
            if self._comm is not None:
                if buf.free_event is not None:
                    self._comm.wait_event(buf.free_event)
            with torch.autograd._unsafe_preserve_version_counter(buf.data):
                if self._use_dist:
                    dist.all_gather_into_tensor(u.full, u.lp_shard, group=self._group)
                else:
                    self.pg.backend().all_gather(u.lp_shard, u.full)
            if self._comm is not None:
                u.gather_event = torch.cuda.Event()
                u.gather_event.record(self._comm)
        if buf.owner is not None and buf.owner is not u:
            buf.owner.gathered = False
        buf.owner = u
        u.gathered = True

    def _wait(self, u: FlatUnit) -> None:
        if u.gather_event is not None:
            torch.cuda.current_stream().wait_event(u.gather_event)
            u.gather_event = None

    def _mark_free(self, u: FlatUnit) -> None:
        if self._comm is not None and u.world > 1:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            u.buffer.free_event = ev

    def _neighbor(self, u: FlatUnit, step: int):
        j = u.index + step
        return self.block_units[j] if 0 <= j < len(self.block_units) else None

    def _pre_forward(self, u: FlatUnit) -> None:
        if self._k4 and not u.gathered and u.world > 1:
            # no gather here: the unit's first Linear gathers inside its own kernel
            u.gate.pending = True
            return
        self._gather(u)
        self._wait(u)
        nxt = self._neighbor(u, -1 if self._phase == "bwd" else 1)
        if nxt is not None and not self._k4:
            self._gather(nxt)

    def _post_forward(self, u: FlatUnit) -> None:
        if self._k4 and getattr(u, "gate", None) is not None and u.gate.pending:
            # nothing in the unit consumed the gate (a unit without a Linear on the kernel path)
            u.gate.pending = False
        self._mark_free(u)

    def _pre_backward(self, u: FlatUnit) -> None:
        self._enter_backward()
        if self._k4 and getattr(u, "gate", None) is not None and u.world > 1:
            if u.gathered:
                u.gate.pending = False
                return
            if u.gate.linear_only:
                # With activation checkpointing the unit's forward is recomputed before any weight is
                # read, and its first Linear gathers inside its kernel; without, the first Linear
                # backward that finds the gate still pending gathers the plain way.
                u.gate.pending = True
                return
        self._gather(u)
        self._wait(u)
        prv = self._neighbor(u, -1)
        if prv is not None and not self._k4:
            self._gather(prv)

    # ------------------------------------------------------------------ gradients
    def _enter_backward(self) -> None:
        if self._phase == "bwd":
            return
        if self._fused is not None and self._sync and self._fused_pending:
            raise RuntimeError(
                "FSDP with the in-backward fused AdamW applies the update inside backward: a second "
                "backward before fused_optimizer().step() would apply a second update. Accumulate "
                "micro-batches under no_sync() and let only the last backward synchronise.")
        self._phase = "bwd"
        for u in self.units:
            u.pending = len(u.params)
            # A reduced gradient of an earlier backward that no zero_grad() has cleared: keep it, the
            # reduction of this backward is added to it (gradient accumulation over micro-batches).
            if self._sync and u.master._axon_grad is not None:
                u._carry = u.master._axon_grad.to(self.device, copy=True)
        torch.autograd.Variable._execution_engine.queue_callback(self._finish_backward)

    def _on_grad(self, u: FlatUnit, idx: int, p) -> None:
        g = p.grad
        if g is None:
            return
        self._enter_backward()
        dst = u.grad_views[idx]
        if u.grad_written[idx]:
            dst.add_(g)
        else:
            dst.copy_(g)
            u.grad_written[idx] = True
        p.grad = None
        if not u.is_root:
            self._arrived(u)

    def _arrived(self, u: FlatUnit) -> None:
        u.pending -= 1
        if u.pending == 0:
            self._mark_free(u)
            if self._sync:
                self._reduce(u)

    def _reduce(self, u: FlatUnit) -> None:
        """Mean over ranks of the unit's flat gradient; this rank keeps its shard."""
        if self.world == 1:
            u.master._axon_grad = u.grad_shard
        elif self._fused is not None and u.world > 1:
            hp = self._fused_hp
            with self._stream_ctx():
                if self._comm is not None:
                    self._comm.wait_stream(torch.cuda.current_stream())
                b1, b2 = hp.get("betas", (0.9, 0.999))
                if self._fused_kind == "lamb":
                    self._lamb_tables(u)
                    self._fused.step_unit_lamb1(u.grad_off, u.shard, u.master.data, u.m1, u.m2, u.upd, u.seg_start,
                                                u.seg_gid, self._lamb_norms, beta1=b1, beta2=b2,
                                                eps=hp.get("eps", 1e-6), wd=hp.get("weight_decay", 0.0),
                                                step=self._fused_step + 1,
                                                bias_correction=hp.get("bias_correction", True))
                else:
                    self._fused.step_unit(u.grad_off, u.shard, u.master.data, u.m1, u.m2, u.lp_shard,
                                          lr=hp["lr"], beta1=b1, beta2=b2, eps=hp.get("eps", 1e-8),
                                          wd=hp.get("weight_decay", 0.01), step=self._fused_step + 1)
        else:
            with self._stream_ctx():
                if self._comm is not None:
                    self._comm.wait_stream(torch.cuda.current_stream())
                if u.world == 1:   # NoShard: all-reduce the whole flat gradient
                    self.pg.backend().all_reduce(u.grad_flat, ReduceOp.Average)
                elif self._use_dist:
                    dist.reduce_scatter_tensor(u.grad_shard, u.grad_flat, op=dist.ReduceOp.AVG,
                                               group=self._group)
                else:
                    self.pg.backend().reduce_scatter(u.grad_flat, u.grad_shard, ReduceOp.Average)
            u.master._axon_grad = u.grad_shard
        if getattr(u, "_carry", None) is not None:
            with self._stream_ctx():
                u.grad_shard.add_(u._carry)
            u._carry = None
        if self._cpu_offload is not CPUOffload.None_:
            # the optimizer steps on the host: hand it the reduced shard there (the copy is ordered
            # after the reduction on the same stream; _finish_backward waits for it)
            with self._stream_ctx():
                u.grad_host.copy_(u.grad_shard, non_blocking=True)
            u.master._axon_grad = u.grad_host
        if self._fused is not None and u.world > 1:
            self._fused_pending = True
        u.grad_written = [False] * len(u.params)
        u.reduced = True

    def _finish_backward(self) -> None:
        if self._sync:
            for u in self.units:
                if not getattr(u, "reduced", False) and any(u.grad_written):
                    self._reduce(u)
            if self._comm is not None:
                torch.cuda.current_stream().wait_stream(self._comm)
            if self._cpu_offload is not CPUOffload.None_ and self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()      # the host reads the gradient copies next
        for u in self.units:
            u.reduced = False
        self._phase = "idle"

    @contextlib.contextmanager
    def no_sync(self):
        """Accumulates gradients locally; the next backward outside the context reduces them.
        Backward calls outside the context accumulate as well (each one is reduced and added to the
        sharded gradient until ``zero_grad``), at the price of one collective per call."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    # ------------------------------------------------------------------ forward
    def forward(self, *args, **kwargs):
        return self._run(self.module, *args, **kwargs)

    def call(self, method: str, *args, **kwargs):
        """Runs ``module.<method>(*args)`` (e.g. ``forward_with_loss``) under the engine."""
        return self._run(getattr(self.module, method), *args, **kwargs)

    def _run(self, fn, *args, **kwargs):
        self._phase = "fwd"
        if self._comm is not None:
            # shards written by the optimizer on the compute stream must be visible to the gathers
            self._comm.wait_stream(torch.cuda.current_stream())
        if self.world > 1:
            for u in self.units:
                if u.world > 1:
                    u.gathered = False
                    if u.buffer.owner is u and self._rotate and not u.is_root:
                        u.buffer.owner = None
        if self.root is not None:
            self._gather(self.root)
            self._wait(self.root)
        if self.block_units and not self._k4:
            self._gather(self.block_units[0])
        out = fn(*args, **kwargs)
        for t in (out if isinstance(out, (tuple, list)) else (out,)):
            if torch.is_tensor(t) and t.requires_grad:
                t.register_hook(lambda g: (self._enter_backward(), g)[1])
        return out

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("module"), name)

    # ------------------------------------------------------------------ reference methods
    def parameters(self, recurse: bool = True):
        """The tensors an optimizer must step: one fp32 master shard per unit."""
        return iter([u.master for u in self.units])

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        return iter([(f"{prefix}{u.name}.flat_shard", u.master) for u in self.units])

    def model_parameters(self):
        return self.module.parameters()

    def gather_parameters(self) -> None:
        for u in self.units:
            if not (self._rotate and not u.is_root):
                self._gather(u)
                self._wait(u)

    def reshard_parameters(self) -> None:
        for u in self.units:
            if u.world > 1:
                u.gathered = False

    def sync_gradients(self) -> None:
        for u in self.units:
            if any(u.grad_written):
                self._reduce(u)
        if self._comm is not None:
            torch.cuda.current_stream().wait_stream(self._comm)
        if self._cpu_offload is not CPUOffload.None_ and self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()

    def zero_grad(self, set_to_none: bool = True) -> None:
        for u in self.units:
            u.master._axon_grad = None
            u._carry = None
            u.grad_written = [False] * len(u.params)
        for p in self.module.parameters():
            p.grad = None

    def clip_grad_norm(self, max_norm: float) -> torch.Tensor:
        """Global L2 norm over all shards (local sum of squares -> all-reduce -> scale;
        fsdp.rs:284-314)."""
        from ..ops import optim as O
        grads = [u.master._axon_grad for u in self.units if u.master._axon_grad is not None]
        if not grads:
            return torch.zeros((), device=self.device)
        ss = O.grad_sumsq(grads)
        if self.world > 1 and self._strategy is not ShardingStrategy.NoShard:
            self.pg.backend().all_reduce(ss, ReduceOp.Sum)
        norm = ss.sqrt()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        if O.supported(grads, grads):
            O.multi_tensor("scale", None, grads, clip_coef=coef)
        else:
            for g in grads:
                g.mul_(coef.to(g.dtype)[0])
        return norm[0]

    def memory_estimate(self) -> FSDPMemoryStats:
        total = sum(u.param_numel() for u in self.units)
        local = sum(u.shard for u in self.units)
        bpe = torch.empty((), dtype=self.param_dtype).element_size()
        return FSDPMemoryStats(total, total * bpe, local, local * (bpe + 4), local * 8,
                               total / max(local, 1), self.world)

    def module_mut(self):
        """The wrapped module (modules are mutable objects: the same object as ``.module``)."""
        return self.module

    def process_group(self):
        return self.pg

    # ------------------------------------------------------------------ state (sharded checkpoints)
    def full_state_dict(self) -> dict:
        """Full-precision state dict of the wrapped module, gathered from the master shards."""
        out = {}
        names = {id(p): n for n, p in self.module.named_parameters()}
        for u in self.units:
            if u.world > 1:
                full = torch.empty(u.padded, dtype=torch.float32, device=self.device)
                self.pg.backend().all_gather(u.master.detach(), full)
            else:
                full = u.master.detach()
            for p, o in zip(u.params, u.offsets):
                out[names[id(p)]] = full[o:o + p.numel()].view(p.shape).clone()
        for n, b in self.module.named_buffers():
            out[n] = b.detach().clone()
        return out

    def load_full_state_dict(self, sd: dict) -> None:
        names = {id(p): n for n, p in self.module.named_parameters()}
        for u in self.units:
            flat = torch.zeros(u.padded, dtype=torch.float32, device=self.device)
            for p, o in zip(u.params, u.offsets):
                flat[o:o + p.numel()].copy_(torch.as_tensor(sd[names[id(p)]]).reshape(-1))
            lo = u.rank * u.shard
            with torch.no_grad():
                u.master.copy_(flat[lo:lo + u.shard])
                u.lp_shard.copy_(flat[lo:lo + u.shard].to(self.param_dtype))
            if u.world > 1:
                u.gathered = False


class _FusedOptimizerHandle:
    def __init__(self, engine: FullyShardedDataParallel):
        self.engine = engine

    def step(self) -> None:
        if self.engine._fused_kind == "lamb" and self.engine._fused is not None:
            self.engine._lamb_phase2()
        self.engine._fused_step += 1
        self.engine._fused_pending = False

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.engine.zero_grad()

    def get_lr(self) -> float: return self.engine._fused_hp["lr"]
    def set_lr(self, lr: float) -> None: self.engine._fused_hp["lr"] = float(lr)


class _GradSink:
    """Lets a GEMM write a weight gradient straight into the unit's flat gradient buffer."""

    def __init__(self, engine: FullyShardedDataParallel, unit: FlatUnit, idx: int):
        self.engine, self.unit, self.idx = engine, unit, idx

    def target(self) -> torch.Tensor:
        return self.unit.grad_views[self.idx]

    def first_write(self) -> bool:
        return not self.unit.grad_written[self.idx]

    def done(self) -> None:
        self.engine._enter_backward()
        self.unit.grad_written[self.idx] = True
        self.engine._arrived(self.unit)


FSDP = FullyShardedDataParallel
