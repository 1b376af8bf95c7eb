"""Bottleneck analysis.

Parity: crates/axonml-profile/src/bottleneck.rs (``BottleneckType``, ``Severity{Low, Medium, High,
Critical}``, ``Bottleneck{bottleneck_type, severity, name, description, suggestion, metrics}``,
``AnalyzerConfig`` with the default thresholds 20 % of the time, 10 000 calls, 30 % of the peak
memory, 1 GFLOPS and leak checking, ``BottleneckAnalyzer::analyze`` sorted by severity).  Severity
steps: a slow operation is Medium from 25 %, High from 35 %, Critical from 50 % of the profiled
time; a call count is Medium from 50 000 and High from 100 000; a memory hotspot is Medium from
45 % and High from 60 %; leaked bytes above 5 % of everything allocated are reported, Medium from
10 %, High from 25 %, Critical from 50 %."""
from __future__ import annotations

import dataclasses
import enum
import functools


class BottleneckType(enum.Enum):
    SlowOperation = "slow_operation"
    HighCallCount = "high_call_count"
    MemoryHotspot = "memory_hotspot"
    LowThroughput = "low_throughput"
    MemoryLeak = "memory_leak"


@functools.total_ordering
class Severity(enum.Enum):
    Low = 1
    Medium = 2
    High = 3
    Critical = 4

    def __lt__(self, other):
        if isinstance(other, Severity):
            return self.value < other.value
        return NotImplemented

    def __float__(self) -> float:
        return self.value / 4.0


def _steps(value: float, *levels) -> Severity:
    """Highest ``Severity`` whose threshold ``value`` reaches; ``levels`` are (threshold, severity) from the top."""
    for threshold, sev in levels:
        if value >= threshold:
            return sev
    return Severity.Low


@dataclasses.dataclass
class Bottleneck:
    kind: BottleneckType
    name: str
    severity: Severity
    description: str
    suggestion: str
    metrics: dict = dataclasses.field(default_factory=dict)

    @property
    def bottleneck_type(self) -> BottleneckType:
        return self.kind


@dataclasses.dataclass
class AnalyzerConfig:
    slow_op_threshold_pct: float = 20.0
    high_call_threshold: int = 10_000
    memory_hotspot_threshold_pct: float = 30.0
    min_gflops_threshold: float = 1.0
    check_memory_leaks: bool = True


class BottleneckAnalyzer:
    def __init__(self, config: AnalyzerConfig | None = None, *, time_threshold: float | None = None, call_threshold: int | None = None,
                 memory_threshold: float | None = None, gflops_threshold: float | None = None):
        c = config or AnalyzerConfig()
        if time_threshold is not None: c.slow_op_threshold_pct = 100.0 * time_threshold
        if call_threshold is not None: c.high_call_threshold = call_threshold
        if memory_threshold is not None: c.memory_hotspot_threshold_pct = 100.0 * memory_threshold
        if gflops_threshold is not None: c.min_gflops_threshold = gflops_threshold
        self.config = c

    @classmethod
    def new(cls): return cls()
    @classmethod
    def with_config(cls, config: AnalyzerConfig): return cls(config)

    def analyze(self, profiler) -> list:
        c, out = self.config, []
        stats = profiler.compute.all_stats()
        total = sum(s.total_ns for s in stats.values())
        for s in stats.values():
            pct = 100.0 * s.total_ns / total if total else 0.0
            if total and pct >= c.slow_op_threshold_pct:
                sev = _steps(pct, (50.0, Severity.Critical), (35.0, Severity.High), (25.0, Severity.Medium))
                out.append(Bottleneck(BottleneckType.SlowOperation, s.name, sev, f"{s.name} takes {pct:.1f}% of the profiled time",
                                      "fuse it with its neighbours or move it onto tensor cores",
                                      {"time_pct": pct, "total_ms": s.total_ns / 1e6, "calls": s.count}))
            if s.count >= c.high_call_threshold:
                sev = _steps(s.count, (100_000, Severity.High), (50_000, Severity.Medium))
                out.append(Bottleneck(BottleneckType.HighCallCount, s.name, sev, f"{s.name} was called {s.count} times",
                                      "batch the calls or capture them in a CUDA graph", {"calls": s.count, "avg_us": s.avg_ns() / 1e3}))
            if s.flops > 0 and s.gflops() < c.min_gflops_threshold:
                out.append(Bottleneck(BottleneckType.LowThroughput, s.name, Severity.Medium, f"{s.name} reaches {s.gflops():.3f} GFLOPS",
                                      "check tiling / occupancy / data layout", {"gflops": s.gflops()}))
        mem = profiler.memory
        base = mem.peak or sum(mem.by_name.values())
        for name, b in mem.by_name.items():
            pct = 100.0 * b / base if base else 0.0
            if base and pct >= c.memory_hotspot_threshold_pct:
                sev = _steps(pct, (60.0, Severity.High), (45.0, Severity.Medium))
                out.append(Bottleneck(BottleneckType.MemoryHotspot, name, sev, f"{name} allocated {pct:.1f}% of the peak memory",
                                      "reuse buffers or shard the tensor", {"bytes": b, "pct_of_peak": pct}))
        if c.check_memory_leaks and mem.total_allocated > mem.total_freed:
            leaked = mem.total_allocated - mem.total_freed
            pct = 100.0 * leaked / mem.total_allocated
            if pct > 5.0:
                sev = _steps(pct, (50.0, Severity.Critical), (25.0, Severity.High), (10.0, Severity.Medium))
                names = sorted({r.name for r in mem.leaks()})
                out.append(Bottleneck(BottleneckType.MemoryLeak, ", ".join(names[:5]) or "memory", sev,
                                      f"{leaked} bytes ({pct:.1f}% of everything allocated) were never freed", "free or pool the buffers",
                                      {"leaked_bytes": leaked, "leak_pct": pct, "live_allocations": len(mem.leaks())}))
        return sorted(out, key=lambda b: b.severity, reverse=True)

    def summary(self, profiler) -> str:
        found = self.analyze(profiler)
        if not found:
            return "No bottlenecks detected."
        return "\n".join(f"[{b.severity.name.upper():8s}] {b.kind.name}: {b.description}\n           -> {b.suggestion}" for b in found)
