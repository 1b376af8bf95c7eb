"""Executable models of the peer-signal protocols of the fused kernels, run under randomised
interleavings on the CPU.

Multi-rank kernels cannot be put under a race detector on the GPU pool, so the protocols are
checked here: every agent (a CTA role of one rank) is a Python generator that yields at each
point where the hardware may switch to another agent (before a flag load, after a remote store
becomes visible, ...).  A seeded scheduler picks the next runnable agent; an agent waiting on a
flag is runnable only when the flag has the value it waits for.  The run fails on

* deadlock: agents remain, none is runnable;
* a read of a staging slot that does not hold this call's data (stale or not yet written);
* an overwrite of a slot whose previous content has not been consumed.

Two protocols are modelled, as the kernels implement them:

* ``reduce_scatter``: ``gemm_comm.cu`` MODE_RS: epoch-valued flags that only grow; a call first
  waits for every peer's "consumed call e-1" signal; partial tiles go to the owner's staging slot
  ring phase by ring phase; flags of a phase are raised after the first tile of the next phase (or
  before the rank's own rows, or at the end); the own rows come last and wait for all peers' flags.
* ``all_reduce``: ``comm.cu`` two-phase all-reduce with a device-side call counter: every block
  signals every peer and waits for theirs (cross-GPU barrier), reduces its slice from all peers'
  buffers, barriers again before the buffers may be reused."""
from __future__ import annotations

import random


class ProtocolError(AssertionError):
    pass


class _Wait:
    """Yielded by an agent: runnable once ``pred()`` holds."""

    def __init__(self, pred, what: str):
        self.pred, self.what = pred, what


def run_agents(agents: dict, seed: int, max_steps: int = 1_000_000) -> int:
    """Runs generators to completion under a random schedule.  Returns the number of steps."""
    rng = random.Random(seed)
    pending = {name: None for name in agents}          # name -> the _Wait it is blocked on (or None)
    live = dict(agents)
    steps = 0
    while live:
        runnable = [n for n in live if pending[n] is None or pending[n].pred()]
        if not runnable:
            blocked = {n: pending[n].what for n in live}
            raise ProtocolError(f"deadlock (seed {seed}): {blocked}")
        n = rng.choice(runnable)
        pending[n] = None
        try:
            y = next(live[n])
        except StopIteration:
            del live[n]
            continue
        if isinstance(y, _Wait):
            pending[n] = y
        steps += 1
        if steps > max_steps:
            raise ProtocolError(f"no progress after {max_steps} steps (seed {seed})")
    return steps


# ------------------------------------------------------------------------------ reduce-scatter
class ReduceScatterModel:
    """W ranks, C CTAs per rank, T tiles per shard; ``calls`` back-to-back launches on the same
    staging buffers and signal words."""

    def __init__(self, world: int, ctas: int, tiles: int, calls: int = 2, defer_flags: bool = True,
                 flush_before_own: bool = True, wait_done: bool = True):
        self.W, self.C, self.T, self.calls = world, ctas, tiles, calls
        self.defer, self.flush_before_own, self.wait_done = defer_flags, flush_before_own, wait_done
        # flags[owner][src][tile] = epoch of the last partial tile that landed; done[rank][peer]
        self.flags = [[[0] * tiles for _ in range(world)] for _ in range(world)]
        self.done = [[0] * world for _ in range(world)]
        self.counter = [0] * world
        # staging[owner][src][tile] = (epoch written, consumed?)
        self.staging = [[[(0, True)] * tiles for _ in range(world)] for _ in range(world)]
        self.out = [[None] * tiles for _ in range(world)]

    def _cta(self, rank: int, cta: int, epoch: int):
        W, C, T = self.W, self.C, self.T
        # start of call: every peer must have consumed the previous call
        for peer in range(W):
            if peer != rank and self.wait_done:
                yield _Wait(lambda p=peer: self.done[rank][p] >= epoch - 1, f"r{rank}c{cta} done[{peer}]>={epoch - 1}")
        pend: list = []
        pend_shard = None

        def release(items):
            for shard, tile in items:
                self.flags[shard][rank][tile] = epoch

        total = W * T
        for t in range(cta, total, C):
            ring_pos, tile = divmod(t, T)
            shard = (rank + 1 + ring_pos) % W
            yield None                                   # the MMA of the tile
            if shard != rank:
                w_epoch, consumed = self.staging[shard][rank][tile]
                if not consumed:
                    raise ProtocolError(f"r{rank} overwrites staging[{shard}][{rank}][{tile}] of call {w_epoch} unconsumed")
                self.staging[shard][rank][tile] = (epoch, False)        # the bulk store lands
                yield None
                if self.defer:
                    if pend and pend_shard != shard:
                        release(pend)
                        pend = []
                    pend_shard = shard
                    pend.append((shard, tile))
                else:
                    release([(shard, tile)])
            else:
                if pend and self.flush_before_own:
                    release(pend)
                    pend = []
                for peer in range(W):
                    if peer != rank:
                        yield _Wait(lambda p=peer, tl=tile: self.flags[rank][p][tl] >= epoch,
                                    f"r{rank}c{cta} flag[{peer}][{tile}]>={epoch}")
                for peer in range(W):
                    if peer != rank:
                        w_epoch, consumed = self.staging[rank][peer][tile]
                        if w_epoch != epoch or consumed:
                            raise ProtocolError(f"r{rank} reads staging[{rank}][{peer}][{tile}]: holds call {w_epoch}, wants {epoch}")
                        self.staging[rank][peer][tile] = (w_epoch, True)
                        yield None
                self.out[rank][tile] = epoch
        if pend:
            release(pend)
        # end of call: the last CTA of the launch tells the peers
        self.counter[rank] += 1
        if self.counter[rank] == epoch * C:
            for peer in range(W):
                if peer != rank:
                    self.done[peer][rank] = epoch

    def _rank_stream(self, rank: int, cta: int):
        for e in range(1, self.calls + 1):
            yield from self._cta(rank, cta, e)

    def run(self, seed: int) -> int:
        agents = {f"r{r}c{c}": self._rank_stream(r, c) for r in range(self.W) for c in range(self.C)}
        steps = run_agents(agents, seed)
        for r in range(self.W):
            if any(o != self.calls for o in self.out[r]):
                raise ProtocolError(f"rank {r} did not finish every own tile: {self.out[r]}")
        return steps


# ------------------------------------------------------------------------------ all-reduce
class AllReduceModel:
    """Two-phase all-reduce over peer-visible buffers: barrier, reduce own slice from every peer,
    write the result to every peer, barrier.  ``skip_second_barrier`` models the bug the second
    barrier prevents (a fast rank overwrites its buffer for call e+1 while a peer still reads e)."""

    def __init__(self, world: int, blocks: int, calls: int = 3, skip_second_barrier: bool = False):
        self.W, self.B, self.calls, self.skip2 = world, blocks, calls, skip_second_barrier
        self.buf = [[0] * blocks for _ in range(world)]             # epoch of the data in slice b of rank r's buffer
        self.sig = [[[0] * world for _ in range(blocks)] for _ in range(world)]   # sig[rank][block][src]
        self.result = [[0] * blocks for _ in range(world)]

    def _barrier(self, rank, b, value):
        for peer in range(self.W):
            self.sig[peer][b][rank] = value
            yield None
        for peer in range(self.W):
            yield _Wait(lambda p=peer: self.sig[rank][b][p] >= value, f"r{rank}b{b} sig[{peer}]>={value}")

    def _block(self, rank: int, b: int):
        for e in range(1, self.calls + 1):
            self.buf[rank][b] = e                                   # the call's input is in place
            yield from self._barrier(rank, b, 2 * e - 1)
            for peer in range(self.W):                              # read the slice from every peer
                if self.buf[peer][b] != e:
                    raise ProtocolError(f"r{rank}b{b} call {e} reads peer {peer} holding call {self.buf[peer][b]}")
                yield None
            self.result[rank][b] = e
            if not self.skip2:
                yield from self._barrier(rank, b, 2 * e)

    def run(self, seed: int) -> int:
        agents = {f"r{r}b{b}": self._block(r, b) for r in range(self.W) for b in range(self.B)}
        steps = run_agents(agents, seed)
        if any(v != self.calls for r in self.result for v in r):
            raise ProtocolError("a block did not finish every call")
        return steps


def check_all(seeds: int = 200) -> dict:
    """The sweep the CPU test runs: every protocol, several shapes, ``seeds`` schedules each."""
    n = 0
    for seed in range(seeds):
        for (w, c, t) in ((2, 2, 3), (3, 4, 5), (4, 3, 4), (8, 2, 2)):
            ReduceScatterModel(w, c, t, calls=2).run(seed)
            n += 1
        for (w, b) in ((2, 2), (4, 3), (8, 2)):
            AllReduceModel(w, b, calls=3).run(seed)
            n += 1
    return {"runs": n, "seeds": seeds}
