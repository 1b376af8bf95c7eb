"""Benchmark helpers (crates/axonml/src/benchmark.rs:45-260, hub.rs:349-414).  Timing uses CUDA
events on the current stream when the model lives on a GPU (after warm-up, synchronised on both
sides) and ``perf_counter`` on CPU; peak memory is what the CUDA allocator reports, not the
reference's ``input_elems * 4 * 3`` guess."""
from __future__ import annotations

import dataclasses
import statistics
import time

import torch


def _is_cuda(model, x) -> bool:
    return torch.is_tensor(x) and x.is_cuda


def warmup_model(model, input, iterations: int = 3) -> None:
    with torch.no_grad():
        for _ in range(iterations):
            model(input)
    if _is_cuda(model, input):
        torch.cuda.synchronize()


class BenchmarkResult:
    def __init__(self, model_name: str, latencies_ms, peak_memory_bytes: int = 0):
        lat = sorted(latencies_ms)
        self.model_name, self.iterations = model_name, len(lat)
        self.mean_ms = statistics.fmean(lat) if lat else 0.0
        self.std_ms = statistics.pstdev(lat) if len(lat) > 1 else 0.0
        self.min_ms, self.max_ms = (lat[0], lat[-1]) if lat else (0.0, 0.0)
        pick = lambda q: lat[min(len(lat) - 1, int(q * len(lat)))] if lat else 0.0
        self.p50_ms, self.p95_ms, self.p99_ms = pick(0.5), pick(0.95), pick(0.99)
        self.throughput = 1000.0 / self.mean_ms if self.mean_ms else 0.0
        self.peak_memory_bytes = peak_memory_bytes

    @classmethod
    def new(cls, model_name, latencies_ms, peak_memory_bytes=0): return cls(model_name, latencies_ms, peak_memory_bytes)

    def print_summary(self) -> None:
        print(f"{self.model_name}: mean {self.mean_ms:.3f} ms (p50 {self.p50_ms:.3f}, p95 {self.p95_ms:.3f}, "
              f"p99 {self.p99_ms:.3f}), {self.throughput:.1f} it/s, peak {self.peak_memory_bytes / 2**20:.1f} MiB")


def benchmark_model(model, input, iterations: int = 100, warmup: int = 3, name: str = "model") -> BenchmarkResult:
    warmup_model(model, input, warmup)
    lat = []
    cuda = _is_cuda(model, input)
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    with torch.no_grad():
        for _ in range(iterations):
            if cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                model(input)
                b.record()
                b.synchronize()
                lat.append(a.elapsed_time(b))
            else:
                t0 = time.perf_counter()
                model(input)
                lat.append((time.perf_counter() - t0) * 1e3)
    peak = torch.cuda.max_memory_allocated() if cuda else input.numel() * input.element_size()
    return BenchmarkResult(name, lat, peak)


def benchmark_model_named(model, input, name: str, iterations: int = 100): return benchmark_model(model, input, iterations, name=name)


def compare_models(models: dict, input, iterations: int = 50) -> list:
    return [benchmark_model(m, input, iterations, name=n) for n, m in models.items()]


def compare_benchmarks(results) -> None:
    base = results[0].mean_ms if results else 1.0
    for r in results:
        print(f"{r.model_name:24s} {r.mean_ms:10.3f} ms  x{base / r.mean_ms if r.mean_ms else 0:.2f}")


@dataclasses.dataclass
class ThroughputConfig:
    batch_sizes: tuple = (1, 4, 8, 16, 32, 64)
    iterations: int = 50
    warmup: int = 3


@dataclasses.dataclass
class ThroughputResult:
    batch_size: int
    mean_ms: float
    samples_per_sec: float


def throughput_test(model, make_input, config: ThroughputConfig | None = None) -> list:
    config = config or ThroughputConfig()
    out = []
    for bs in config.batch_sizes:
        r = benchmark_model(model, make_input(bs), config.iterations, config.warmup)
        out.append(ThroughputResult(bs, r.mean_ms, bs * 1000.0 / r.mean_ms if r.mean_ms else 0.0))
    return out


def print_throughput_results(results) -> None:
    for r in results:
        print(f"batch {r.batch_size:4d}: {r.mean_ms:9.3f} ms  {r.samples_per_sec:12.1f} samples/s")


@dataclasses.dataclass
class MemorySnapshot:
    parameter_bytes: int
    buffer_bytes: int
    gradient_bytes: int
    num_parameters: int

    def total_mb(self) -> float: return (self.parameter_bytes + self.buffer_bytes + self.gradient_bytes) / 2**20


def profile_model_memory(model) -> MemorySnapshot:
    pb = sum(p.numel() * p.element_size() for p in model.parameters())
    bb = sum(b.numel() * b.element_size() for b in model.buffers())
    gb = sum(p.numel() * p.element_size() for p in model.parameters() if p.requires_grad)
    return MemorySnapshot(pb, bb, gb, sum(p.numel() for p in model.parameters()))


def print_memory_profile(snapshot: MemorySnapshot, name: str) -> None:
    print(f"{name}: {snapshot.num_parameters} parameters, {snapshot.total_mb():.2f} MiB "
          f"(params {snapshot.parameter_bytes}, buffers {snapshot.buffer_bytes}, grads {snapshot.gradient_bytes})")
