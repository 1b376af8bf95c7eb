"""Inference metrics (crates/axonml-server/src/inference/metrics.rs:19-240, api/metrics.rs:32-71):
per-endpoint success/error counts, latency ring with p50/p95/p99, histogram buckets, requests per
second, error rate, a request timer, and Prometheus text exposition."""
from __future__ import annotations

import collections
import threading
import time

BUCKETS_MS = (1, 5, 10, 25, 50, 100, 250, 500, 1000, 2500, 5000, 10000)


class EndpointMetrics:
    def __init__(self, name: str, ring: int = 1000):
        self.name = name
        self.success = self.errors = 0
        self.latencies = collections.deque(maxlen=ring)
        self.histogram = [0] * (len(BUCKETS_MS) + 1)
        self.total_latency_ms = 0.0
        self.started = time.time()
        self.gauges: dict = {}

    def record(self, latency_ms: float, ok: bool = True) -> None:
        if ok:
            self.success += 1
        else:
            self.errors += 1
        self.latencies.append(latency_ms)
        self.total_latency_ms += latency_ms
        for i, b in enumerate(BUCKETS_MS):
            if latency_ms <= b:
                self.histogram[i] += 1
                break
        else:
            self.histogram[-1] += 1

    def total(self) -> int: return self.success + self.errors
    def error_rate(self) -> float: return self.errors / self.total() if self.total() else 0.0
    def rps(self) -> float: return self.total() / max(time.time() - self.started, 1e-9)
    def mean_ms(self) -> float: return self.total_latency_ms / self.total() if self.total() else 0.0

    def percentile(self, p: float) -> float:
        if not self.latencies:
            return 0.0
        s = sorted(self.latencies)
        return s[min(len(s) - 1, int(p / 100.0 * len(s)))]

    def p50(self): return self.percentile(50)
    def p95(self): return self.percentile(95)
    def p99(self): return self.percentile(99)

    def snapshot(self) -> dict:
        return {"endpoint": self.name, "success": self.success, "errors": self.errors, "error_rate": self.error_rate(),
                "rps": self.rps(), "mean_ms": self.mean_ms(), "p50_ms": self.p50(), "p95_ms": self.p95(),
                "p99_ms": self.p99(), "histogram": dict(zip([str(b) for b in BUCKETS_MS] + ["+Inf"], self.histogram)),
                **self.gauges}


class RequestTimer:
    def __init__(self, metrics: "InferenceMetrics", endpoint: str):
        self.metrics, self.endpoint, self.t0 = metrics, endpoint, time.perf_counter()
    def finish_success(self) -> float: return self._finish(True)
    def finish_error(self) -> float: return self._finish(False)
    def _finish(self, ok):
        ms = (time.perf_counter() - self.t0) * 1e3
        self.metrics.record(self.endpoint, ms, ok)
        return ms


class InferenceMetrics:
    def __init__(self):
        self._lock = threading.Lock()
        self.endpoints: dict[str, EndpointMetrics] = {}

    @classmethod
    def new(cls): return cls()

    def endpoint(self, name: str) -> EndpointMetrics:
        with self._lock:
            if name not in self.endpoints:
                self.endpoints[name] = EndpointMetrics(name)
            return self.endpoints[name]

    def record(self, name: str, latency_ms: float, ok: bool = True) -> None:
        e = self.endpoint(name)
        with self._lock:
            e.record(latency_ms, ok)

    def set_gauge(self, name: str, key: str, value: float) -> None:
        self.endpoint(name).gauges[key] = value

    def time_request(self, name: str) -> RequestTimer: return RequestTimer(self, name)
    def snapshot(self) -> dict: return {k: v.snapshot() for k, v in self.endpoints.items()}

    def prometheus(self, extra: dict | None = None) -> str:
        lines = ['# TYPE axonml_server_info gauge', 'axonml_server_info{version="0.1.0"} 1']
        for k, v in (extra or {}).items():
            lines += [f"# TYPE axonml_{k} gauge", f"axonml_{k} {v}"]
        for n, e in self.endpoints.items():
            lab = f'{{endpoint="{n}"}}'
            lines += [f"axonml_requests_total{lab} {e.total()}", f"axonml_request_errors_total{lab} {e.errors}",
                      f"axonml_request_latency_ms_p50{lab} {e.p50():.3f}", f"axonml_request_latency_ms_p95{lab} {e.p95():.3f}",
                      f"axonml_request_latency_ms_p99{lab} {e.p99():.3f}", f"axonml_requests_per_second{lab} {e.rps():.3f}"]
            cum = 0
            for b, c in zip(list(BUCKETS_MS) + ["+Inf"], e.histogram):
                cum += c
                lines.append(f'axonml_request_latency_ms_bucket{{endpoint="{n}",le="{b}"}} {cum}')
            for k, v in e.gauges.items():
                lines.append(f"axonml_{k}{lab} {v}")
        return "\n".join(lines) + "\n"
