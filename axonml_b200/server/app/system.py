"""System information for the platform server and the CLI: host, memory, GPUs (NVML through
``pynvml`` when the driver is there, else ``torch.cuda``), a realtime sample with a short history
and a small compute/copy benchmark.

Parity: ``/api/system/info``, ``/api/system/gpus``, ``/api/system/metrics`` with history,
``/api/system/benchmark`` (crates/axonml-server/src/api/system.rs); the reference enumerates
adapters through wgpu, here the device layer is CUDA + NVML.  Nothing in this module changes a GPU
setting: it only reads."""
from __future__ import annotations

import collections
import os
import platform
import threading
import time


def _nvml():
    try:
        import pynvml
        pynvml.nvmlInit()
        return pynvml
    except Exception:  # noqa: BLE001 - no driver, no library: fall back to torch
        return None


def list_gpus() -> list[dict]:
    out = []
    nv = _nvml()
    if nv is not None:
        try:
            for i in range(nv.nvmlDeviceGetCount()):
                h = nv.nvmlDeviceGetHandleByIndex(i)
                mem = nv.nvmlDeviceGetMemoryInfo(h)
                name = nv.nvmlDeviceGetName(h)
                d = {"id": i, "name": name.decode() if isinstance(name, bytes) else name, "backend": "cuda",
                     "memory_total": int(mem.total), "memory_used": int(mem.used), "memory_free": int(mem.free)}
                for key, fn in (("utilization", lambda: nv.nvmlDeviceGetUtilizationRates(h).gpu),
                                ("temperature", lambda: nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU)),
                                ("power_w", lambda: nv.nvmlDeviceGetPowerUsage(h) / 1000.0),
                                ("sm_clock_mhz", lambda: nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))):
                    try:
                        d[key] = fn()
                    except Exception:  # noqa: BLE001 - a counter the board does not expose
                        d[key] = None
                out.append(d)
            return out
        except Exception:  # noqa: BLE001
            out = []
    try:
        import torch
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                p = torch.cuda.get_device_properties(i)
                free, total = torch.cuda.mem_get_info(i)
                out.append({"id": i, "name": p.name, "backend": "cuda", "memory_total": total, "memory_used": total - free,
                            "memory_free": free, "compute_capability": f"{p.major}.{p.minor}",
                            "multiprocessors": p.multi_processor_count, "utilization": None, "temperature": None,
                            "power_w": None, "sm_clock_mhz": None})
    except Exception:  # noqa: BLE001
        pass
    return out


def _meminfo() -> dict:
    d = {}
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                k, v = line.split(":", 1)
                d[k] = int(v.split()[0]) * 1024
    except OSError:
        pass
    return d


def system_info() -> dict:
    mi = _meminfo()
    try:
        import torch
        torch_v, cuda_v = torch.__version__, torch.version.cuda
    except Exception:  # noqa: BLE001
        torch_v = cuda_v = None
    gpus = list_gpus()
    return {"platform": platform.system(), "arch": platform.machine(), "hostname": platform.node(),
            "python": platform.python_version(), "cpu_count": os.cpu_count(), "total_memory_bytes": mi.get("MemTotal"),
            "available_memory_bytes": mi.get("MemAvailable"), "torch": torch_v, "cuda": cuda_v, "gpus": gpus,
            "gpu_count": len(gpus), "framework": "axonml_b200"}


def _cpu_times():
    try:
        with open("/proc/stat") as f:
            v = [int(x) for x in f.readline().split()[1:8]]
        return sum(v), v[3] + v[4]
    except (OSError, ValueError):
        return 0, 0


class SystemMonitor:
    """Samples on demand; keeps the last ``history`` samples for the dashboard's charts."""

    def __init__(self, history: int = 300):
        self._hist = collections.deque(maxlen=history)
        self._last = _cpu_times()
        self._lock = threading.Lock()

    def sample(self) -> dict:
        tot, idle = _cpu_times()
        with self._lock:
            dt, di = tot - self._last[0], idle - self._last[1]
            self._last = (tot, idle)
        mi = _meminfo()
        s = {"timestamp": time.time(), "cpu_percent": round(100.0 * (1 - di / dt), 2) if dt > 0 else 0.0,
             "memory_used_bytes": (mi.get("MemTotal", 0) - mi.get("MemAvailable", 0)) or None,
             "memory_total_bytes": mi.get("MemTotal"),
             "load_avg": list(os.getloadavg()) if hasattr(os, "getloadavg") else None,
             "gpus": [{k: g.get(k) for k in ("id", "utilization", "memory_used", "memory_total", "temperature", "power_w",
                                             "sm_clock_mhz")} for g in list_gpus()]}
        with self._lock:
            self._hist.append(s)
        return s

    def history(self) -> list[dict]:
        with self._lock:
            return list(self._hist)

    def correlation(self) -> dict:
        """Pairs (cpu %, memory used, first GPU utilisation) over the history, for the scatter chart."""
        h = self.history()
        return {"points": [{"cpu": s["cpu_percent"], "memory": s["memory_used_bytes"],
                            "gpu": (s["gpus"][0]["utilization"] if s["gpus"] else None), "t": s["timestamp"]} for s in h]}


def run_benchmark(size: int = 1024, iters: int = 5, device: str | None = None) -> dict:
    """Matmul throughput and copy bandwidth, CPU or one GPU (the reference's hardware benchmark
    measures a naive matmul and a memcpy, crates/axonml-cli/src/commands/bench.rs:543-640)."""
    import torch
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    a, b = torch.randn(size, size, device=dev, dtype=dt), torch.randn(size, size, device=dev, dtype=dt)

    def timed(fn):
        fn()
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        return (time.perf_counter() - t0) / iters

    t_mm = timed(lambda: a @ b)
    src = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    dst = torch.empty_like(src)
    t_cp = timed(lambda: dst.copy_(src))
    return {"device": str(dev), "dtype": str(dt).replace("torch.", ""), "matmul_size": size,
            "matmul_gflops": 2.0 * size ** 3 / t_mm / 1e9, "copy_gb_per_s": 2 * src.numel() / t_cp / 1e9}
