"""Pipeline parallelism with real GPipe and 1F1B schedules.

Reference API (crates/axonml-distributed/src/pipeline.rs:31-375): ``PipelineSchedule`` {GPipe,
OneFOneBSchedule (default), InterleavedOneFOneB}, ``PipelineStage{module, stage_id, device_rank}``,
``Pipeline.from_modules(mods, pg).schedule(s).num_microbatches(n)``, ``forward`` (micro-batched,
activations sent stage to stage), ``PipelineMemoryStats``.  The reference runs GPipe forward only
and has no backward scheduling (pipeline.rs:235-245); here ``train_step`` runs forward and backward
of every microbatch in schedule order, with activations and their gradients exchanged by
point-to-point send/recv of the process group (NCCL p2p on GPUs, posted asynchronously so that a
transfer overlaps the next microbatch's compute)."""
from __future__ import annotations

import dataclasses
import enum

import torch

from ..nn.module import Module
from .process_group import ProcessGroup


class PipelineSchedule(enum.Enum):
    GPipe = "gpipe"
    OneFOneBSchedule = "1f1b"
    InterleavedOneFOneB = "interleaved_1f1b"


@dataclasses.dataclass
class PipelineStage:
    module: torch.nn.Module
    stage_id: int
    device_rank: int


@dataclasses.dataclass
class PipelineMemoryStats:
    num_stages: int
    num_microbatches: int
    peak_activations_per_stage: int
    schedule: PipelineSchedule


class Pipeline(Module):
    def __init__(self, stages, process_group: ProcessGroup, schedule=PipelineSchedule.OneFOneBSchedule,
                 num_microbatches: int = 1):
        super().__init__()
        self.stages = list(stages)
        self.pg = process_group
        self._schedule, self._m = schedule, num_microbatches
        self.local = torch.nn.ModuleList([s.module for s in self.stages
                                          if s.device_rank == self.pg.rank() and s.module is not None])
        self._shape_cache = {}
        self._pending = []

    def _drain(self) -> None:
        for work, _ in self._pending:
            work.wait()
        self._pending = []

    @classmethod
    def from_modules(cls, modules, process_group: ProcessGroup):
        w = process_group.world_size()
        return cls([PipelineStage(m, i, i % w) for i, m in enumerate(modules)], process_group)

    def schedule(self, s: PipelineSchedule): self._schedule = s; return self
    def num_microbatches(self, n: int): self._m = n; return self
    def num_stages(self) -> int: return len(self.stages)
    def get_schedule(self) -> PipelineSchedule: return self._schedule

    def memory_stats(self) -> PipelineMemoryStats:
        S, M = len(self.stages), self._m
        peak = S * M if self._schedule is PipelineSchedule.GPipe else min(S, M)
        return PipelineMemoryStats(S, M, peak, self._schedule)

    # ------------------------------------------------------------------ helpers
    def split_microbatches(self, x: torch.Tensor): return list(x.chunk(self._m, dim=0))
    def combine_microbatches(self, outs): return torch.cat(list(outs), dim=0)

    def _my_stage(self):
        mine = [s for s in self.stages if s.device_rank == self.pg.rank()]
        if len(mine) != 1:
            raise ValueError("train_step expects exactly one stage per rank (use interleaving via stage lists)")
        return mine[0]

    def _send(self, t: torch.Tensor, dst: int, tag: int) -> None:
        meta = torch.tensor([t.dim()] + list(t.shape) + [0] * (7 - t.dim()), dtype=torch.int64, device=t.device)
        key = (dst, tag & 1)
        be = self.pg.backend()
        if key not in self._shape_cache:
            be.send(meta, dst, 1000 + (tag & 1))
            self._shape_cache[key] = tuple(t.shape)
        t = t.contiguous()
        if hasattr(be, "isend"):
            # posted asynchronously: a blocking send could deadlock against the peer's own send in
            # the steady 1F1B phase, and the transfer overlaps the next microbatch's compute
            self._pending.append((be.isend(t, dst, tag & 1), t))
        else:
            be.send(t, dst, tag & 1)

    def _recv(self, src: int, tag: int, dtype, device) -> torch.Tensor:
        key = (-src - 1, tag & 1)
        if key not in self._shape_cache:
            meta = torch.zeros(8, dtype=torch.int64, device=device)
            self.pg.backend().recv(meta, src, 1000 + (tag & 1))
            m = meta.tolist()
            self._shape_cache[key] = tuple(m[1:1 + m[0]])
        out = torch.empty(self._shape_cache[key], dtype=dtype, device=device)
        self.pg.backend().recv(out, src, tag & 1)
        return out

    # ------------------------------------------------------------------ forward only (reference semantics)
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Micro-batched forward through all stages; the last stage's rank returns the combined
        output, other ranks return their last local activation."""
        outs = []
        for mb in self.split_microbatches(x):
            h = mb
            for st in self.stages:
                if st.device_rank == self.pg.rank():
                    if st.stage_id > 0 and self.stages[st.stage_id - 1].device_rank != self.pg.rank():
                        h = self._recv(self.stages[st.stage_id - 1].device_rank, 0, x.dtype if x.is_floating_point() else torch.float32, x.device)
                    h = st.module(h)
                    nxt = st.stage_id + 1
                    if nxt < len(self.stages) and self.stages[nxt].device_rank != self.pg.rank():
                        self._send(h, self.stages[nxt].device_rank, 0)
            outs.append(h)
        self._drain()
        return self.combine_microbatches(outs)

    # ------------------------------------------------------------------ training schedules
    def train_step(self, inputs: torch.Tensor | None, targets: torch.Tensor | None, loss_fn,
                   act_dtype=torch.float32) -> torch.Tensor | None:
        """One forward+backward over ``num_microbatches`` microbatches.  ``inputs`` are used by the
        first stage, ``targets`` and ``loss_fn(output, target)`` by the last; gradients accumulate
        in the stage's parameters.  Returns the mean loss on the last stage, None elsewhere."""
        st = self._my_stage()
        S, M, sid = len(self.stages), self._m, st.stage_id
        first, last = sid == 0, sid == S - 1
        prev_rank = self.stages[sid - 1].device_rank if not first else None
        next_rank = self.stages[sid + 1].device_rank if not last else None
        dev = next(st.module.parameters()).device
        in_mbs = self.split_microbatches(inputs) if first else [None] * M
        tg_mbs = self.split_microbatches(targets) if last else [None] * M
        saved, losses = {}, []

        def fwd(i):
            if first:
                x = in_mbs[i]
            else:
                x = self._recv(prev_rank, 0, act_dtype, dev).requires_grad_(True)
            y = st.module(x)
            if last:
                loss = loss_fn(y, tg_mbs[i]) / M
                losses.append(loss.detach())
                saved[i] = (x, loss)
            else:
                self._send(y.detach(), next_rank, 0)
                saved[i] = (x, y)

        def bwd(i):
            x, y = saved.pop(i)
            if last:
                y.backward()
            else:
                g = self._recv(next_rank, 1, y.dtype, dev)
                y.backward(g)
            if not first:
                self._send(x.grad, prev_rank, 1)

        if self._schedule is PipelineSchedule.GPipe:
            for i in range(M):
                fwd(i)
            for i in reversed(range(M)):
                bwd(i)
        else:
            warm = min(S - sid - 1, M)
            for i in range(warm):
                fwd(i)
            f, b = warm, 0
            while f < M:
                fwd(f)
                f += 1
                bwd(b)
                b += 1
            while b < M:
                bwd(b)
                b += 1
        self._drain()
        return torch.stack(losses).sum() if last else None
