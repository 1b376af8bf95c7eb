"""Pipeline parallelism with real GPipe and 1F1B schedules.

Reference API (crates/axonml-distributed/src/pipeline.rs:31-375): ``PipelineSchedule`` {GPipe,
OneFOneBSchedule (default), InterleavedOneFOneB}, ``PipelineStage{module, stage_id, device_rank}``,
``Pipeline.from_modules(mods, pg).schedule(s).num_microbatches(n)``, ``forward`` (micro-batched,
activations sent stage to stage), ``PipelineMemoryStats``.  The reference runs GPipe forward only
and has no backward scheduling (pipeline.rs:235-245); here ``train_step`` runs forward and backward
of every microbatch in schedule order, with activations and their gradients exchanged by
point-to-point send/recv of the process group (NCCL p2p on GPUs, posted asynchronously so that a
transfer overlaps the next microbatch's compute).  ``InterleavedOneFOneB`` gives every rank several
model chunks (stage i lives on rank i mod W) and runs them from a static schedule that every rank
derives identically (``build_schedule``); receives are posted one operation ahead of their use.
``Pipeline.last_comm`` reports how long the last step waited for transfers against how long it
computed."""
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

    def forward(self, x):
        return self.module(x)

    __call__ = forward


@dataclasses.dataclass
class PipelineMemoryStats:
    num_stages: int
    num_microbatches: int
    peak_activations_per_stage: int
    schedule: PipelineSchedule

    @staticmethod
    def gpipe_peak_activations(num_stages: int, num_microbatches: int) -> int:
        """GPipe keeps every microbatch's activations on every stage until the backward pass."""
        return num_stages * num_microbatches

    @staticmethod
    def one_f_one_b_peak_activations(num_stages: int, num_microbatches: int) -> int:
        """1F1B holds at most as many microbatches in flight as there are stages."""
        return min(num_stages, num_microbatches)


def build_schedule(num_stages: int, world: int, num_microbatches: int, in_flight_limit=None):
    """Static pipeline schedule for stages laid out round-robin over ``world`` ranks (stage s on rank
    s mod world, so a rank holds num_stages / world model chunks).  Returns ``{rank: [(kind, stage,
    microbatch)]}`` with kind "F" or "B", the order in which each rank runs its operations.

    The lists come from a time-stepped simulation that every rank can repeat bit for bit: in each
    slot a rank runs one ready operation, a backward before a forward (1F1B), forwards in the
    interleaved order of groups of ``world`` microbatches per chunk, while the forwards a rank has
    in flight stay under its limit (the interleaved warm-up depth (world - rank - 1) * 2 +
    (chunks - 1) * world, plus one).  Two messages between the same pair of ranks in the same
    direction are consumed in the order they were sent, so transports that match messages by order
    (NCCL) see the same sequence on both sides."""
    S, W, M = num_stages, world, num_microbatches
    V = (S + W - 1) // W
    rank_of = lambda s: s % W
    done_at: dict = {}                       # (kind, stage, mb) -> slot it ran in
    order = {r: [] for r in range(W)}
    queues: dict = {}                        # (src rank, dst rank, kind) -> [(stage of consumer, mb)] in send order
    in_flight = {r: 0 for r in range(W)}
    # one chunk per rank: the classic 1F1B depth (a rank keeps world - rank forwards in flight)
    default = lambda r: (W - r) if V == 1 else (W - r - 1) * 2 + (V - 1) * W + 1
    limit = {r: (in_flight_limit if in_flight_limit is not None else default(r)) for r in range(W)}
    total = 2 * S * M
    slot = 0

    def fkey(s, m): return (m // W, s // W, m % W)
    def bkey(s, m): return (m // W, -(s // W), m % W)

    while len(done_at) < total:
        ran = []
        for r in range(W):
            cands = []
            for s in range(r, S, W):
                for m in range(M):
                    if ("B", s, m) not in done_at and ("F", s, m) in done_at and done_at[("F", s, m)] < slot:
                        dep = ("B", s + 1, m)
                        if s == S - 1 or (dep in done_at and done_at[dep] < slot):
                            if s < S - 1 and rank_of(s + 1) != r:
                                q = queues.get((rank_of(s + 1), r, "B"), [])
                                if not q or q[0] != (s, m):
                                    continue
                            cands.append((0, bkey(s, m), "B", s, m))
                    if ("F", s, m) not in done_at and in_flight[r] < limit[r]:
                        dep = ("F", s - 1, m)
                        if s == 0 or (dep in done_at and done_at[dep] < slot):
                            if s > 0 and rank_of(s - 1) != r:
                                q = queues.get((rank_of(s - 1), r, "F"), [])
                                if not q or q[0] != (s, m):
                                    continue
                            cands.append((1, fkey(s, m), "F", s, m))
            if cands:
                _, _, kind, s, m = min(cands)
                ran.append((r, kind, s, m))
        if not ran:
            if slot > 4 * total + 16:
                raise RuntimeError("pipeline schedule did not converge")
            slot += 1
            continue
        for r, kind, s, m in ran:
            done_at[(kind, s, m)] = slot
            order[r].append((kind, s, m))
            if kind == "F":
                in_flight[r] += 1
                if s > 0 and rank_of(s - 1) != r:
                    queues[(rank_of(s - 1), r, "F")].pop(0)
                if s < S - 1 and rank_of(s + 1) != r:
                    queues.setdefault((r, rank_of(s + 1), "F"), []).append((s + 1, m))
            else:
                in_flight[r] -= 1
                if s < S - 1 and rank_of(s + 1) != r:
                    queues[(rank_of(s + 1), r, "B")].pop(0)
                if s > 0 and rank_of(s - 1) != r:
                    queues.setdefault((r, rank_of(s - 1), "B"), []).append((s - 1, m))
        slot += 1
    return order


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
        self.last_comm = None        # set by the scheduled (interleaved) path after every step

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
        W = max(1, self.pg.world_size())
        if self._schedule is PipelineSchedule.GPipe:
            peak = S * M
        elif self._schedule is PipelineSchedule.InterleavedOneFOneB and S > W:
            peak = min((W - 1) * 2 + ((S + W - 1) // W - 1) * W + 1, S // W * M)
        else:
            peak = min(S, M)
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
        mine = [x for x in self.stages if x.device_rank == self.pg.rank()]
        if self._schedule is PipelineSchedule.InterleavedOneFOneB or len(mine) != 1:
            return self._train_step_scheduled(inputs, targets, loss_fn, act_dtype)
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

    # ------------------------------------------------------------------ scheduled execution (several stages per rank)
    def _train_step_scheduled(self, inputs, targets, loss_fn, act_dtype):
        """Runs this rank's operations in the order of ``build_schedule``.  Activations travel to
        the next stage's rank, gradients back; a transfer to a stage on the same rank is a plain
        hand-over.  The receive of the next operation is posted before the current one computes."""
        import time
        S, M, W, me = len(self.stages), self._m, self.pg.world_size(), self.pg.rank()
        for st in self.stages:
            if st.device_rank != st.stage_id % W:
                raise ValueError("scheduled execution expects stage i on rank i mod world (Pipeline.from_modules)")
        ops = build_schedule(S, W, M)[me]
        mods = {st.stage_id: st.module for st in self.stages if st.device_rank == me}
        dev = next(next(iter(mods.values())).parameters()).device
        in_mbs = self.split_microbatches(inputs) if 0 in mods else None
        tg_mbs = self.split_microbatches(targets) if (S - 1) in mods else None
        be = self.pg.backend()
        can_post = hasattr(be, "irecv")
        local: dict = {}            # hand-overs between stages of this rank: (kind, stage, mb) -> tensor
        saved: dict = {}
        losses = []
        posted: dict = {}           # index of the operation -> (work, buffer) of its pre-posted receive
        wait_s = compute_s = 0.0

        def source(kind, s):
            """Rank the input of operation (kind, s) comes from, or None (first stage forward, last
            stage backward, or the producer lives on this rank)."""
            src = s - 1 if kind == "F" else s + 1
            if src < 0 or src >= S or src % W == me:
                return None
            return src % W

        def post(i):
            if i >= len(ops) or i in posted or not can_post:
                return
            kind, s, m = ops[i]
            src = source(kind, s)
            key = (-src - 1, 0 if kind == "F" else 1) if src is not None else None
            if src is None or key not in self._shape_cache:
                return                                  # the first message of a channel carries its shape: blocking path
            buf = torch.empty(self._shape_cache[key], dtype=act_dtype, device=dev)
            posted[i] = (be.irecv(buf, src, 0 if kind == "F" else 1), buf)

        def receive(i, kind, s):
            nonlocal wait_s
            src = source(kind, s)
            if src is None:
                return None
            t0 = time.perf_counter()
            if i in posted:
                work, buf = posted.pop(i)
                work.wait()
            else:
                buf = self._recv(src, 0 if kind == "F" else 1, act_dtype, dev)
            wait_s += time.perf_counter() - t0
            return buf

        for i, (kind, s, m) in enumerate(ops):
            if kind == "F":
                if s == 0:
                    x = in_mbs[m]
                elif (s - 1) % W == me:
                    x = local.pop(("F", s, m)).requires_grad_(True)
                else:
                    x = receive(i, kind, s).requires_grad_(True)
                post(i + 1)         # after this operation's own receive: receives keep the order of the sends
                t0 = time.perf_counter()
                y = mods[s](x)
                if s == S - 1:
                    loss = loss_fn(y, tg_mbs[m]) / M
                    losses.append(loss.detach())
                    saved[(s, m)] = (x, loss)
                else:
                    saved[(s, m)] = (x, y)
                compute_s += time.perf_counter() - t0
                if s < S - 1:
                    if (s + 1) % W == me:
                        local[("F", s + 1, m)] = y.detach()
                    else:
                        self._send(y.detach(), (s + 1) % W, 0)
            else:
                x, y = saved.pop((s, m))
                if s == S - 1:
                    g = None
                elif (s + 1) % W == me:
                    g = local.pop(("B", s, m))
                else:
                    g = receive(i, kind, s)
                post(i + 1)
                t0 = time.perf_counter()
                y.backward(g) if g is not None else y.backward()
                compute_s += time.perf_counter() - t0
                if s > 0:
                    if (s - 1) % W == me:
                        local[("B", s - 1, m)] = x.grad
                    else:
                        self._send(x.grad, (s - 1) % W, 1)
        self._drain()
        self.last_comm = {"wait_s": wait_s, "compute_s": compute_s,
                          "overlap": 1.0 - wait_s / max(wait_s + compute_s, 1e-9), "operations": len(ops)}
        return torch.stack(losses).sum() if losses else None
