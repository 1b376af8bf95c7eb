"""CPU-vs-GPU correctness harness (crates/axonml-core/src/backends/gpu_tests.rs:28-733):
``GpuTestConfig`` (atol 1e-5, rtol 1e-4, sizes 1..4096), LCG ``random_vec`` (seeds 42/123),
``assert_close``, CPU references, ``run_all_tests`` and a report printer."""
from __future__ import annotations

import dataclasses

import torch

from .backends import CpuBackend, CudaBackend


@dataclasses.dataclass
class GpuTestConfig:
    atol: float = 1e-5
    rtol: float = 1e-4
    test_sizes: tuple = (1, 7, 16, 64, 256, 1024, 4096)
    benchmark_sizes: tuple = (1024, 16384, 262144, 1048576)
    warmup_iters: int = 5
    bench_iters: int = 100


@dataclasses.dataclass
class GpuTestResult:
    name: str
    passed: bool
    max_error: float = 0.0
    message: str = ""
    throughput_gbps: float | None = None
    latency_us: float | None = None

    # the reference's builders (gpu_tests.rs:79-113); ``pass`` is a keyword, hence the underscore
    @classmethod
    def pass_(cls, name: str): return cls(name, True)
    @classmethod
    def fail(cls, name: str, error: str): return cls(name, False, 0.0, error)

    def with_error(self, max_abs_error: float):
        self.max_error = float(max_abs_error)
        return self

    def with_perf(self, throughput_gbps: float, latency_us: float):
        self.throughput_gbps, self.latency_us = float(throughput_gbps), float(latency_us)
        return self

    @property
    def error(self): return self.message or None
    @property
    def max_abs_error(self): return self.max_error


@dataclasses.dataclass
class GpuTestReport:
    results: list = dataclasses.field(default_factory=list)
    backend: str = "cuda"
    capabilities: object = None

    @classmethod
    def new(cls, backend: str): return cls([], backend)

    def with_capabilities(self, caps):
        self.capabilities = caps
        return self

    def add(self, r: GpuTestResult) -> None: self.results.append(r)
    add_result = add
    def passed(self) -> int: return sum(r.passed for r in self.results)
    def failed(self) -> int: return sum(not r.passed for r in self.results)
    passed_count, failed_count = passed, failed
    def all_passed(self) -> bool: return self.failed() == 0

    def print_summary(self) -> None:
        print(f"GPU Test Report: {self.backend}")
        if self.capabilities is not None:
            c = self.capabilities
            print(f"Device: {c.name}  memory {c.total_memory / 2 ** 30:.1f} GiB  SMs {getattr(c, 'sm_count', 0)}")
        for r in self.results:
            perf = f" {r.throughput_gbps:.1f} GB/s {r.latency_us:.1f} us" if r.throughput_gbps is not None else ""
            print(f"[{'PASS' if r.passed else 'FAIL'}] {r.name} max_err={r.max_error:.3e}{perf} {r.message}")
        print(f"{self.passed()} passed, {self.failed()} failed")


def random_vec(n: int, seed: int) -> torch.Tensor:
    """Deterministic LCG in [-1, 1) (gpu_tests.rs:252-262)."""
    out = torch.empty(n)
    s = seed & 0xFFFFFFFFFFFFFFFF
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = ((s >> 33) / float(1 << 31)) * 2.0 - 1.0
    return out


def assert_close(a: torch.Tensor, b: torch.Tensor, atol: float, rtol: float):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    ok = bool((err <= atol + rtol * b.abs()).all())
    return ok, float(err.max()) if err.numel() else 0.0


def run_all_tests(config: GpuTestConfig | None = None, backend: CudaBackend | None = None) -> GpuTestReport:
    cfg, rep = config or GpuTestConfig(), GpuTestReport()
    be = backend or CudaBackend(0)
    if not be.is_available():
        rep.add(GpuTestResult("cuda_available", True, 0.0, "skipped: no CUDA device"))
        return rep
    dev = be.device().to_torch()
    cases = [("add", lambda a, b: be.add_f32(a, b), CpuBackend.add, False), ("sub", lambda a, b: be.sub_f32(a, b), CpuBackend.sub, False),
             ("mul", lambda a, b: be.mul_f32(a, b), CpuBackend.mul, False),
             ("relu", lambda a, b: be.relu_f32(a), lambda a, b: CpuBackend.relu(a), False),
             ("sigmoid", lambda a, b: be.sigmoid_f32(a), lambda a, b: CpuBackend.sigmoid(a), True),
             ("tanh", lambda a, b: be.tanh_f32(a), lambda a, b: CpuBackend.tanh(a), True),
             ("gelu", lambda a, b: be.gelu_f32(a), lambda a, b: CpuBackend.gelu(a), True)]
    for name, gpu_fn, cpu_fn, approx in cases:
        for n in cfg.test_sizes:
            a, b = random_vec(n, 42), random_vec(n, 123)
            got = gpu_fn(a.to(dev), b.to(dev))
            ok, err = assert_close(got, cpu_fn(a, b), 1e-3 if approx else cfg.atol, 1e-2 if approx else cfg.rtol)
            rep.add(GpuTestResult(f"{name}_{n}", ok, err))
    for m, k, n in ((4, 8, 4), (64, 64, 64), (128, 256, 64)):
        a, b = random_vec(m * k, 42).view(m, k), random_vec(k * n, 123).view(k, n)
        ok, err = assert_close(be.gemm_f32(a.to(dev), b.to(dev)), CpuBackend.matmul(a, b), 1e-3, 1e-2)
        rep.add(GpuTestResult(f"gemm_{m}x{k}x{n}", ok, err))
    return rep
