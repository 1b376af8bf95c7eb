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
import enum
import json
import threading
import time

import torch


class ProfileError(Exception):
    """Errors of the profiler (crates/axonml-profile/src/error.rs:10-30)."""


class OperationNotFound(ProfileError, KeyError):
    def __init__(self, name):
        super().__init__(f"Operation not found: {name}")

    def __str__(self) -> str: return self.args[0]


class InvalidState(ProfileError, RuntimeError):
    def __init__(self, what): super().__init__(f"Invalid profiler state: {what}")


class ProfileIoError(ProfileError, OSError):
    def __init__(self, what): super().__init__(f"IO error: {what}")


class ProfileSerializationError(ProfileError, ValueError):
    def __init__(self, what): super().__init__(f"Serialization error: {what}")


class TimerError(ProfileError):
    def __init__(self, what): super().__init__(f"Timer error: {what}")


def format_duration(ns: float) -> str:
    """ns / us / ms / s with three significant decimals (compute.rs:240-255)."""
    for unit, div in (("s", 1e9), ("ms", 1e6), ("us", 1e3)):
        if ns >= div:
            return f"{ns / div:.3f} {unit}"
    return f"{ns:.0f} ns"


def format_bytes(n: int) -> str:
    """B / KB / MB / GB in powers of 1024 (memory.rs:190-205)."""
    for unit, div in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if n >= div:
            return f"{n / div:.2f} {unit}"
    return f"{n} B"


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
    # the reference's accessor names (compute.rs:30-62); times in seconds
    def avg_time(self) -> float: return self.avg_ns() / 1e9
    def total_time(self) -> float: return self.total_ns / 1e9
    def min_time(self) -> float: return (self.min_ns if self.count else 0.0) / 1e9
    def max_time(self) -> float: return self.max_ns / 1e9
    def bandwidth_gbps(self) -> float: return self.gbps()


@dataclasses.dataclass
class ProfiledOp:
    """An operation that has been started and not yet stopped (compute.rs:75-84)."""
    name: str
    start: object                 # perf_counter_ns value on the host, a CUDA event on the device
    flops: float | None = None
    bytes: int | None = None
    on_device: bool = False


class ComputeProfiler:
    def __init__(self):
        self.stats: dict[str, OperationStats] = {}
        self._open: dict[str, list] = {}
        self._pending: list = []

    def start(self, name: str, flops: float | None = None, nbytes: int | None = None) -> None:
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            op = ProfiledOp(name, ev, flops, nbytes, True)
        else:
            op = ProfiledOp(name, time.perf_counter_ns(), flops, nbytes, False)
        self._open.setdefault(name, []).append(op)

    def start_with_flops(self, name: str, flops: float) -> None: self.start(name, flops=flops)
    def start_with_bytes(self, name: str, nbytes: int) -> None: self.start(name, nbytes=nbytes)

    def active(self) -> list:
        """Operations started and not yet stopped."""
        return [op for stack in self._open.values() for op in stack]

    def stop(self, name: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
        stack = self._open.get(name)
        if not stack:
            return
        op = stack.pop()
        flops = flops or op.flops or 0.0
        nbytes = nbytes or op.bytes or 0.0
        if op.on_device:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pending.append((name, op.start, ev, flops, nbytes))
        else:
            self.record(name, time.perf_counter_ns() - op.start, flops, nbytes)

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

    def get_stats(self, name: str):
        self.resolve()
        return self.stats.get(name)

    def require_stats(self, name: str) -> OperationStats:
        s = self.get_stats(name)
        if s is None:
            raise OperationNotFound(name)
        return s

    def all_stats(self) -> dict:
        self.resolve()
        return dict(self.stats)

    def total_time(self, name: str) -> float:
        s = self.get_stats(name)
        return s.total_time() if s else 0.0

    def avg_time(self, name: str) -> float:
        s = self.get_stats(name)
        return s.avg_time() if s else 0.0

    def top(self, n: int = 10):
        self.resolve()
        return sorted(self.stats.values(), key=lambda s: -s.total_ns)[:n]

    top_by_time = top

    def top_by_calls(self, n: int = 10):
        self.resolve()
        return sorted(self.stats.values(), key=lambda s: -s.count)[:n]

    format_duration = staticmethod(format_duration)

    def reset(self) -> None:
        self.stats, self._open, self._pending = {}, {}, []


@dataclasses.dataclass
class AllocationRecord:
    name: str
    size: int
    timestamp: int                # ns since the profiler was created
    freed: bool = False


@dataclasses.dataclass
class MemoryStats:
    current_usage: int = 0
    peak_usage: int = 0
    total_allocated: int = 0
    total_freed: int = 0
    allocation_count: int = 0
    deallocation_count: int = 0
    per_name_usage: dict = dataclasses.field(default_factory=dict)


class MemoryProfiler:
    def __init__(self):
        self.current = self.peak = self.total_allocated = self.total_freed = 0
        self.allocation_count = self.deallocation_count = 0
        self.live: dict = {}
        self.by_name: dict = {}             # bytes ever allocated under a name
        self.records: list[AllocationRecord] = []
        self._usage: dict = {}              # bytes currently held under a name
        self._t0 = time.perf_counter_ns()

    def record_alloc(self, name: str, nbytes: int, ident=None) -> None:
        self.current += nbytes
        self.total_allocated += nbytes
        self.allocation_count += 1
        self.peak = max(self.peak, self.current)
        rec = AllocationRecord(name, nbytes, time.perf_counter_ns() - self._t0)
        self.records.append(rec)
        self.live[ident if ident is not None else (name, len(self.records))] = (name, nbytes, rec)
        self.by_name[name] = self.by_name.get(name, 0) + nbytes
        self._usage[name] = self._usage.get(name, 0) + nbytes

    def record_free(self, name: str, nbytes: int, ident=None) -> None:
        self.current = max(self.current - nbytes, 0)
        self.total_freed += nbytes
        self.deallocation_count += 1
        self._usage[name] = max(self._usage.get(name, 0) - nbytes, 0)
        key = ident if ident is not None and ident in self.live else next(
            (k for k, (n, b, _) in self.live.items() if n == name and b == nbytes), None)
        if key is not None:
            self.live.pop(key)[2].freed = True

    def current_usage(self) -> int: return self.current
    def peak_usage(self) -> int: return self.peak

    def stats(self) -> MemoryStats:
        return MemoryStats(self.current, self.peak, self.total_allocated, self.total_freed, self.allocation_count,
                           self.deallocation_count, {k: v for k, v in self._usage.items() if v})

    def leaks(self) -> list:
        """Allocations never freed, as ``AllocationRecord``s in allocation order."""
        return [r for r in self.records if not r.freed]

    def device_stats(self) -> dict:
        if not torch.cuda.is_available():
            return {}
        return {"allocated": torch.cuda.memory_allocated(), "reserved": torch.cuda.memory_reserved(),
                "peak_allocated": torch.cuda.max_memory_allocated()}

    format_bytes = staticmethod(format_bytes)

    def reset(self) -> None: self.__init__()


class EventType(enum.Enum):
    Start = "B"
    End = "E"
    Instant = "i"
    Alloc = "alloc"
    Free = "free"
    Custom = "custom"


@dataclasses.dataclass
class Event:
    name: str
    event_type: EventType
    timestamp_ns: int
    thread_id: int | None = None
    metadata: str | None = None

    # names of the earlier record type
    @property
    def phase(self) -> str: return self.event_type.value if self.event_type in (EventType.Start, EventType.End) else "i"
    @property
    def ts_us(self) -> float: return self.timestamp_ns / 1e3
    @property
    def tid(self) -> int: return self.thread_id or 0


TimelineEvent = Event


class TimelineProfiler:
    def __init__(self, max_events: int = 100_000):
        self._events: list[Event] = []
        self.max_events = max_events
        self.dropped = 0
        self._t0 = time.perf_counter_ns()

    @classmethod
    def with_capacity(cls, max_events: int): return cls(max_events)

    def record(self, name: str, event_type: EventType, metadata: str | None = None) -> None:
        if len(self._events) >= self.max_events:
            self.dropped += 1               # the timeline keeps its first max_events events
            return
        self._events.append(Event(name, event_type, time.perf_counter_ns() - self._t0, threading.get_ident() & 0xFFFF, metadata))

    def record_with_metadata(self, name: str, event_type: EventType, metadata: str) -> None:
        self.record(name, event_type, metadata)

    def start(self, name: str) -> None: self.record(name, EventType.Start)
    def end(self, name: str) -> None: self.record(name, EventType.End)
    def instant(self, name: str) -> None: self.record(name, EventType.Instant)
    begin = start

    @property
    def events(self) -> list: return self._events
    def events_by_name(self, name: str) -> list: return [e for e in self._events if e.name == name]
    def events_by_type(self, event_type: EventType) -> list: return [e for e in self._events if e.event_type is event_type]
    def event_count(self) -> int: return len(self._events)

    def duration(self, name: str) -> float | None:
        """Seconds from the first Start to the last End of ``name``; None when either is missing."""
        starts = [e.timestamp_ns for e in self._events if e.name == name and e.event_type is EventType.Start]
        ends = [e.timestamp_ns for e in self._events if e.name == name and e.event_type is EventType.End]
        if not starts or not ends or ends[-1] < starts[0]:
            return None
        return (ends[-1] - starts[0]) / 1e9

    def total_duration(self) -> float:
        return (self._events[-1].timestamp_ns - self._events[0].timestamp_ns) / 1e9 if self._events else 0.0

    def to_chrome_trace(self) -> str:
        out = []
        for e in self._events:
            ph = e.phase
            d = {"name": e.name, "ph": ph, "ts": e.ts_us, "pid": 1, "tid": e.tid}
            if ph == "i":
                d["s"] = "g"
            if e.metadata is not None or e.event_type in (EventType.Alloc, EventType.Free, EventType.Custom):
                d["args"] = {"type": e.event_type.name, **({"metadata": e.metadata} if e.metadata is not None else {})}
            out.append(d)
        return json.dumps({"traceEvents": out})

    def to_json(self) -> str:
        return json.dumps([{"name": e.name, "event_type": e.event_type.name, "timestamp_ns": e.timestamp_ns, "thread_id": e.thread_id,
                            "metadata": e.metadata} for e in self._events])

    def export_chrome_trace(self, path) -> None:
        try:
            with open(path, "w") as f:
                f.write(self.to_chrome_trace())
        except OSError as e:
            raise ProfileIoError(str(e)) from e

    def reset(self) -> None: self.__init__(self.max_events)


class Profiler:
    def __init__(self):
        self.memory, self.compute, self.timeline = MemoryProfiler(), ComputeProfiler(), TimelineProfiler()
        self.enabled = True

    @classmethod
    def new(cls): return cls()
    def enable(self) -> None: self.enabled = True
    def disable(self) -> None: self.enabled = False
    def is_enabled(self) -> bool: return self.enabled
    def set_enabled(self, enabled: bool) -> None: self.enabled = bool(enabled)
    def peak_memory(self) -> int: return self.memory.peak_usage()
    def current_memory(self) -> int: return self.memory.current_usage()
    def total_time(self, name: str) -> float: return self.compute.total_time(name)
    def avg_time(self, name: str) -> float: return self.compute.avg_time(name)

    def summary(self):
        """The report of everything recorded so far (``print_summary`` prints it)."""
        return self.report()

    def analyze_bottlenecks(self) -> list:
        from .bottleneck import BottleneckAnalyzer
        return BottleneckAnalyzer().analyze(self)

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

    def record_alloc(self, name, nbytes):
        if self.enabled:
            self.memory.record_alloc(name, nbytes)
            self.timeline.record(name, EventType.Alloc, str(nbytes))

    def record_free(self, name, nbytes):
        if self.enabled:
            self.memory.record_free(name, nbytes)
            self.timeline.record(name, EventType.Free, str(nbytes))
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


# the global profiler's entry points as plain functions (crates/axonml-profile/src/lib.rs:216-233)
def start(name: str) -> None: global_profiler().start(name)
def stop(name: str) -> None: global_profiler().stop(name)
def record_alloc(name: str, nbytes: int) -> None: global_profiler().record_alloc(name, nbytes)
def record_free(name: str, nbytes: int) -> None: global_profiler().record_free(name, nbytes)


class TimingGuard(contextlib.AbstractContextManager):
    """Times one operation on a ``ComputeProfiler`` from construction to ``drop()`` or the end of
    the ``with`` block (compute.rs:255-275)."""

    def __init__(self, profiler: ComputeProfiler, name: str):
        self.profiler, self.name, self._live = profiler, name, True
        profiler.start(name)

    @classmethod
    def new(cls, profiler, name): return cls(profiler, name)

    def drop(self) -> None:
        if self._live:
            self._live = False
            self.profiler.stop(self.name)

    def __exit__(self, *exc):
        self.drop()
        return False
