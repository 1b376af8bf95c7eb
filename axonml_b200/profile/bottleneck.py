"""Bottleneck analysis (crates/axonml-profile/src/bottleneck.rs:74-135)."""
from __future__ import annotations

import dataclasses
import enum


class BottleneckType(enum.Enum):
    SlowOperation = "slow_operation"
    HighCallCount = "high_call_count"
    MemoryHotspot = "memory_hotspot"
    LowThroughput = "low_throughput"
    MemoryLeak = "memory_leak"


@dataclasses.dataclass
class Bottleneck:
    kind: BottleneckType
    name: str
    severity: float
    description: str
    suggestion: str


class BottleneckAnalyzer:
    def __init__(self, time_threshold: float = 0.20, call_threshold: int = 10_000,
                 memory_threshold: float = 0.30, gflops_threshold: float = 1.0):
        self.time_threshold, self.call_threshold = time_threshold, call_threshold
        self.memory_threshold, self.gflops_threshold = memory_threshold, gflops_threshold

    @classmethod
    def new(cls): return cls()

    def analyze(self, profiler) -> list:
        out = []
        total = profiler.compute.total_time_ns() or 1.0
        for s in profiler.compute.stats.values():
            frac = s.total_ns / total
            if frac > self.time_threshold:
                out.append(Bottleneck(BottleneckType.SlowOperation, s.name, frac,
                                      f"{s.name} takes {100 * frac:.1f}% of the profiled time",
                                      "fuse it with its neighbours or move it onto tensor cores"))
            if s.count > self.call_threshold:
                out.append(Bottleneck(BottleneckType.HighCallCount, s.name, min(1.0, s.count / (10 * self.call_threshold)),
                                      f"{s.name} was called {s.count} times", "batch the calls or capture them in a CUDA graph"))
            if s.flops > 0 and s.gflops() < self.gflops_threshold:
                out.append(Bottleneck(BottleneckType.LowThroughput, s.name, 0.5,
                                      f"{s.name} reaches {s.gflops():.3f} GFLOPS", "check tiling / occupancy / data layout"))
        mem_total = sum(profiler.memory.by_name.values()) or 1
        for name, b in profiler.memory.by_name.items():
            if b / mem_total > self.memory_threshold:
                out.append(Bottleneck(BottleneckType.MemoryHotspot, name, b / mem_total,
                                      f"{name} allocated {100 * b / mem_total:.1f}% of all bytes", "reuse buffers or shard the tensor"))
        for name, b in profiler.memory.leaks():
            out.append(Bottleneck(BottleneckType.MemoryLeak, name, 0.3, f"{name}: {b} bytes never freed", "free or pool the buffer"))
        return sorted(out, key=lambda x: -x.severity)
