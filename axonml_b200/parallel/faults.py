"""Host-side fault injection and failure detection.

Nothing here touches a GPU: faults are made on the host (a message that is dropped, delayed or
corrupted; a rank that stops taking part), and failures are detected on the host (a timeout of the
blocking call, a checksum that does not match, a heartbeat that stops).  Device-side waits are
bounded separately and report through the kernel status word (``_native.check_status``).

* ``FaultPlan`` – what to inject, keyed by (operation, sequence number) or (src, dst, tag); handed
  to ``MockBackend.create_world(..., plan=...)`` or wrapped around any backend with ``FaultyBackend``.
* ``Heartbeat`` / ``FailureDetector`` – every rank touches ``hb_<rank>`` in a shared directory from
  a daemon thread; the detector names the ranks whose file is older than the timeout, so the
  survivors learn of a dead rank *before* their next launch instead of inside a collective.
* ``run_with_recovery`` – the recovery policy of this framework: catch the failure, rebuild the
  world from the surviving ranks, reload the last sharded checkpoint (which reshards on load) and
  continue.

The reference has none of this: its ``barrier`` cannot block and a missing message leaves the
receive buffer untouched (crates/axonml-distributed/src/backend.rs:362-386)."""
from __future__ import annotations

import dataclasses
import os
import threading
import time
import zlib

import torch

from .backend import Backend, CommTimeout


class RankKilled(RuntimeError):
    """Raised inside the rank that the plan kills (its thread or process then ends)."""


class CorruptPayload(RuntimeError):
    """A received payload does not match the checksum its sender attached."""


@dataclasses.dataclass
class FaultPlan:
    drop: set = dataclasses.field(default_factory=set)          # {(src, dst, tag, nth)}
    corrupt: set = dataclasses.field(default_factory=set)       # {(src, dst, tag, nth)}
    delay: dict = dataclasses.field(default_factory=dict)       # {(rank, op, nth): seconds}
    kill: dict = dataclasses.field(default_factory=dict)        # {rank: (op, nth)}: the rank raises before that call

    def drop_message(self, src: int, dst: int, tag: int = 0, nth: int = 0) -> "FaultPlan":
        self.drop.add((src, dst, tag, nth)); return self

    def corrupt_message(self, src: int, dst: int, tag: int = 0, nth: int = 0) -> "FaultPlan":
        self.corrupt.add((src, dst, tag, nth)); return self

    def delay_rank(self, rank: int, op: str, nth: int, seconds: float) -> "FaultPlan":
        self.delay[(rank, op, nth)] = seconds; return self

    def kill_rank(self, rank: int, op: str = "all_reduce", nth: int = 0) -> "FaultPlan":
        self.kill[rank] = (op, nth); return self


def checksum(t: torch.Tensor) -> int:
    return zlib.crc32(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes())


class FaultyBackend(Backend):
    """Applies a ``FaultPlan`` in front of another backend (mock, gloo or NCCL: the plan only acts
    on the host side of each call).  With ``verify=True`` every point-to-point payload travels with
    a CRC32 in a second message and the receiver checks it."""

    def __init__(self, inner: Backend, plan: FaultPlan, verify: bool = False):
        self.inner, self.plan, self.verify = inner, plan, verify
        self._count: dict = {}

    def name(self) -> str: return self.inner.name() + "+faults"
    def rank(self) -> int: return self.inner.rank()
    def world_size(self) -> int: return self.inner.world_size()
    def device(self): return self.inner.device() if hasattr(self.inner, "device") else torch.device("cpu")

    def _enter(self, op: str) -> int:
        n = self._count.get(op, 0)
        self._count[op] = n + 1
        r = self.rank()
        if self.plan.kill.get(r) == (op, n):
            raise RankKilled(f"rank {r} killed by the fault plan before {op} #{n}")
        d = self.plan.delay.get((r, op, n))
        if d:
            time.sleep(d)
        return n

    # collectives: kill / delay only (a collective has no single message to drop)
    def all_reduce(self, data, op=None):
        self._enter("all_reduce")
        return self.inner.all_reduce(data, op) if op is not None else self.inner.all_reduce(data)

    def broadcast(self, data, src=0):
        self._enter("broadcast"); return self.inner.broadcast(data, src)

    def all_gather(self, send, recv):
        self._enter("all_gather"); return self.inner.all_gather(send, recv)

    def reduce_scatter(self, send, recv, op=None):
        self._enter("reduce_scatter")
        return self.inner.reduce_scatter(send, recv, op) if op is not None else self.inner.reduce_scatter(send, recv)

    def gather(self, send, recv, dst=0):
        self._enter("gather"); return self.inner.gather(send, recv, dst)

    def scatter(self, send, recv, src=0):
        self._enter("scatter"); return self.inner.scatter(send, recv, src)

    def reduce(self, data, dst=0, op=None):
        self._enter("reduce")
        return self.inner.reduce(data, dst, op) if op is not None else self.inner.reduce(data, dst)

    def barrier(self):
        self._enter("barrier"); return self.inner.barrier()

    # point to point: drop / corrupt as well
    def send(self, data, dst, tag=0):
        self._enter("send")
        key_n = self._count.get(("msg", dst, tag), 0)
        self._count[("msg", dst, tag)] = key_n + 1
        key = (self.rank(), dst, tag, key_n)
        crc = checksum(data) if self.verify else None
        if key in self.plan.drop:
            return
        payload = data
        if key in self.plan.corrupt:
            payload = data.detach().clone()
            flat = payload.view(-1)
            flat[0] = flat[0] + 1 if flat.dtype.is_floating_point else flat[0] ^ 1
        self.inner.send(payload, dst, tag)
        if self.verify:
            self.inner.send(torch.tensor([crc], dtype=torch.int64, device=data.device), dst, tag + (1 << 20))

    def recv(self, data, src, tag=0):
        self._enter("recv")
        self.inner.recv(data, src, tag)
        if self.verify:
            c = torch.zeros(1, dtype=torch.int64, device=data.device)
            self.inner.recv(c, src, tag + (1 << 20))
            if int(c.item()) != checksum(data):
                raise CorruptPayload(f"rank {self.rank()}: payload from {src} (tag {tag}) fails its checksum")

    def new_group(self, ranks):
        g = self.inner.new_group(ranks)
        return None if g is None else FaultyBackend(g, self.plan, self.verify)


# ------------------------------------------------------------------------------ heartbeats
class Heartbeat:
    """Touches ``<dir>/hb_<rank>`` every ``interval_s`` from a daemon thread until ``stop()``."""

    def __init__(self, directory: str, rank: int, interval_s: float = 0.2):
        self.path, self.interval = os.path.join(directory, f"hb_{rank}"), interval_s
        os.makedirs(directory, exist_ok=True)
        self._stop = threading.Event()
        self._beat()
        self._t = threading.Thread(target=self._run, daemon=True, name=f"heartbeat-{rank}")
        self._t.start()

    def _beat(self) -> None:
        with open(self.path, "w") as f:
            f.write(repr(time.time()))

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            self._beat()

    def stop(self) -> None:
        self._stop.set()
        self._t.join(2.0)


class FailureDetector:
    def __init__(self, directory: str, world_size: int, timeout_s: float = 1.0):
        self.dir, self.world, self.timeout = directory, world_size, timeout_s

    def last_seen(self, rank: int) -> float | None:
        try:
            with open(os.path.join(self.dir, f"hb_{rank}")) as f:
                return float(f.read() or 0.0)
        except (OSError, ValueError):
            return None

    def dead_ranks(self) -> list[int]:
        now = time.time()
        out = []
        for r in range(self.world):
            t = self.last_seen(r)
            if t is None or now - t > self.timeout:
                out.append(r)
        return out

    def check(self) -> None:
        """Call between steps, before the next launch: raises if a peer is gone."""
        dead = self.dead_ranks()
        if dead:
            raise CommTimeout(f"ranks {dead} stopped sending heartbeats (timeout {self.timeout}s)")


def run_with_recovery(step_fn, rebuild_fn, max_restarts: int = 3):
    """``step_fn()`` runs the training loop and returns its result; on ``CommTimeout`` /
    ``CorruptPayload`` the loop state is rebuilt by ``rebuild_fn(attempt, error)`` (new world from
    the survivors, last checkpoint reloaded) and the loop starts again."""
    attempt = 0
    while True:
        try:
            return step_fn()
        except (CommTimeout, CorruptPayload) as e:
            attempt += 1
            if attempt > max_restarts:
                raise
            rebuild_fn(attempt, e)
