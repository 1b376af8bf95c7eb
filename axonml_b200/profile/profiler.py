"""Profiler (crates/axonml-profile/src/lib.rs:57-230, compute.rs, memory.rs, timeline.rs,
bottleneck.rs, report.rs): ``Profiler{memory, compute, timeline}``, ``ProfileGuard`` /
``profile_scope``, a global singleton, FLOP/byte annotations (-> GFLOPS, GB/s), memory
alloc/free/peak/leak tracking, Chrome-trace export (always compiled in), bottleneck analysis with
the reference's thresholds (20 % of time, 10 k calls, 30 % of memory, < 1 GFLOPS) and text / JSON /
Markdown / HTML reports.  On CUDA a range is timed with a pair of CUDA events on the current
stream (resolved lazily at report time, so profiling adds no synchronisation) and mirrored as an
NVTX range."""
from __future__ import annotations

import contextlib
import dataclasses
import json
import threading
import time

import torch


@dataclasses.dataclass
class OperationStats:
    name: str
    count: int = 0
    total_ns: float = 0.0
    min_ns: float = float("inf")
    max_ns: float = 0.0
    flops: float = 0.0
    bytes: float = 0.0

    def avg_ns(self) -> float: return self.total_ns / self.count if self.count else 0.0
    def gflops(self) -> float: return self.flops / self.total_ns if self.total_ns else 0.0
    def gbps(self) -> float: return self.bytes / self.total_ns if self.total_ns else 0.0


class ComputeProfiler:
    def __init__(self):
        self.stats: dict[str, OperationStats] = {}
        self._open: dict[str, list] = {}
        self._pending: list = []

    def start(self, name: str) -> None:
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open.setdefault(name, []).append(("cuda", ev))
        else:
            self._open.setdefault(name, []).append(("cpu", time.perf_counter_ns()))

    def stop(self, name: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
        stack = self._open.get(name)
        if not stack:
            return
        kind, t0 = stack.pop()
        if kind == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pending.append((name, t0, ev, flops, nbytes))
        else:
            self.record(name, time.perf_counter_ns() - t0, flops, nbytes)

    def record(self, name: str, ns: float, flops: float = 0.0, nbytes: float = 0.0) -> None:
        s = self.stats.setdefault(name, OperationStats(name))
        s.count += 1
        s.total_ns += ns
        s.min_ns, s.max_ns = min(s.min_ns, ns), max(s.max_ns, ns)
        s.flops += flops
        s.bytes += nbytes

    def resolve(self) -> None:
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b, fl, by in self._pending:
                self.record(name, a.elapsed_time(b) * 1e6, fl, by)
            self._pending = []

    def total_time_ns(self) -> float:
        self.resolve()
        return sum(s.total_ns for s in self.stats.values())

    def top(self, n: int = 10):
        self.resolve()
        return sorted(self.stats.values(), key=lambda s: -s.total_ns)[:n]

    def reset(self) -> None:
        self.stats, self._open, self._pending = {}, {}, []


class MemoryProfiler:
    def __init__(self):
        self.current = self.peak = self.total_allocated = self.total_freed = 0
        self.live: dict = {}
        self.by_name: dict = {}

    def record_alloc(self, name: str, nbytes: int, ident=None) -> None:
        self.current += nbytes
        self.total_allocated += nbytes
        self.peak = max(self.peak, self.current)
        self.live[ident if ident is not None else (name, len(self.live))] = (name, nbytes)
        self.by_name[name] = self.by_name.get(name, 0) + nbytes

    def record_free(self, name: str, nbytes: int, ident=None) -> None:
        self.current -= nbytes
        self.total_freed += nbytes
        if ident is not None:
            self.live.pop(ident, None)
        else:
            for k, (n, b) in list(self.live.items()):
                if n == name and b == nbytes:
                    del self.live[k]
                    break

    def leaks(self): return list(self.live.values())
    def device_stats(self) -> dict:
        if not torch.cuda.is_available():
            return {}
        return {"allocated": torch.cuda.memory_allocated(), "reserved": torch.cuda.memory_reserved(),
                "peak_allocated": torch.cuda.max_memory_allocated()}
    def reset(self) -> None: self.__init__()


@dataclasses.dataclass
class TimelineEvent:
    name: str
    phase: str       # "B" begin, "E" end, "i" instant
    ts_us: float
    tid: int


class TimelineProfiler:
    def __init__(self):
        self.events: list[TimelineEvent] = []
        self._t0 = time.perf_counter_ns()

    def _now(self) -> float: return (time.perf_counter_ns() - self._t0) / 1e3
    def begin(self, name: str) -> None: self.events.append(TimelineEvent(name, "B", self._now(), threading.get_ident() & 0xFFFF))
    def end(self, name: str) -> None: self.events.append(TimelineEvent(name, "E", self._now(), threading.get_ident() & 0xFFFF))
    def instant(self, name: str) -> None: self.events.append(TimelineEvent(name, "i", self._now(), threading.get_ident() & 0xFFFF))

    def to_chrome_trace(self) -> str:
        return json.dumps({"traceEvents": [{"name": e.name, "ph": e.phase, "ts": e.ts_us, "pid": 1, "tid": e.tid,
                                            **({"s": "g"} if e.phase == "i" else {})} for e in self.events]})

    def export_chrome_trace(self, path) -> None:
        with open(path, "w") as f:
            f.write(self.to_chrome_trace())

    def reset(self) -> None: self.__init__()


class Profiler:
    def __init__(self):
        self.memory, self.compute, self.timeline = MemoryProfiler(), ComputeProfiler(), TimelineProfiler()
        self.enabled = True

    @classmethod
    def new(cls): return cls()
    def enable(self) -> None: self.enabled = True
    def disable(self) -> None: self.enabled = False
    def is_enabled(self) -> bool: return self.enabled

    def start(self, name: str) -> None:
        if not self.enabled:
            return
        self.compute.start(name)
        self.timeline.begin(name)
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.nvtx.range_push(name)

    def stop(self, name: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
        if not self.enabled:
            return
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.nvtx.range_pop()
        self.compute.stop(name, flops, nbytes)
        self.timeline.end(name)

    def record_alloc(self, name, nbytes): self.memory.record_alloc(name, nbytes)
    def record_free(self, name, nbytes): self.memory.record_free(name, nbytes)
    def reset(self) -> None:
        self.memory.reset(); self.compute.reset(); self.timeline.reset()

    def scope(self, name: str, flops: float = 0.0, nbytes: float = 0.0): return ProfileGuard(self, name, flops, nbytes)
    def report(self):
        from .report import ProfileReport
        return ProfileReport.generate(self)
    def print_summary(self) -> None: print(self.report().to_text())


class ProfileGuard(contextlib.AbstractContextManager):
    def __init__(self, profiler: Profiler, name: str, flops: float = 0.0, nbytes: float = 0.0):
        self.p, self.name, self.flops, self.nbytes = profiler, name, flops, nbytes
    def __enter__(self):
        self.p.start(self.name)
        return self
    def __exit__(self, *exc):
        self.p.stop(self.name, self.flops, self.nbytes)
        return False


_GLOBAL = None
_LOCK = threading.Lock()


def global_profiler() -> Profiler:
    global _GLOBAL
    with _LOCK:
        if _GLOBAL is None:
            _GLOBAL = Profiler()
        return _GLOBAL


def profile_scope(name: str, flops: float = 0.0, nbytes: float = 0.0) -> ProfileGuard:
    return global_profiler().scope(name, flops, nbytes)
