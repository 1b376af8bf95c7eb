"""ctypes bindings of the in-tree native libraries.

``cuda()`` returns the handle of ``libaxonml_cuda.so`` (hand-written sm_100a kernels) and
``host()`` the handle of ``libaxonml_host.so`` (C++ runtime: codecs, quantisers, CPU reference
kernels).  Both are built on first use if the shared object is missing.  On a machine with a GPU
a missing CUDA library is an error, never a silent fallback to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LOCK = threading.Lock()
_CUDA = None
_HOST = None
_LIBDIR = Path(__file__).resolve().parent / "_lib"

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_int64 = ctypes.c_int64


class NativeError(RuntimeError):
    """Raised when a native launcher returns a non-zero code."""


def _load(name: str, builder: str):
    path = _LIBDIR / name
    if not path.exists() or os.environ.get("AXONML_REBUILD") == "1":
        from . import _build
        getattr(_build, builder)(verbose=True)
    return ctypes.CDLL(str(path))


class _CountingLib:
    """Forwards attribute access to the ctypes library and counts calls of the kernel launchers
    (every ``ax_*`` entry that takes a stream launches at least one kernel)."""

    _NO_LAUNCH = {"ax_version", "ax_sm_count", "ax_norm_bwd_groups", "ax_multi_tensor_limits", "ax_gemm_comm_set_trace",
                  "ax_flash_fwd_set_trace", "ax_gemm_comm_signal_slots", "ax_norm_bwd_noalloc_limits", "ax_gemm_set_pair_mode", "ax_flash_fwd_set_one_tile", "ax_bounds_enabled", "ax_bounds_read", "ax_gemm_pair_capacity"}

    def __init__(self, lib):
        self._lib = lib
        self._cache = {}
        self.launches = 0

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._lib, name)
            if name in self._NO_LAUNCH:
                fn = raw
            else:
                def fn(*args, _raw=raw):
                    self.launches += 1
                    return _raw(*args)
            self._cache[name] = fn
        return fn


def bounds_build() -> bool:
    """``AXONML_BOUNDS=1`` selects the debug build of the kernels whose index checks report a wrong
    index (``bounds_report``) instead of using it."""
    return os.environ.get("AXONML_BOUNDS") == "1"


def cuda():
    """Handle of the CUDA kernel library (built for sm_100a)."""
    global _CUDA
    if _CUDA is None:
        with _LOCK:
            if _CUDA is None:
                if bounds_build():
                    path = _LIBDIR / "libaxonml_cuda_bounds.so"
                    if not path.exists() or os.environ.get("AXONML_REBUILD") == "1":
                        from . import _build
                        _build.build_cuda(verbose=True, bounds=True)
                    _CUDA = _CountingLib(ctypes.CDLL(str(path)))
                else:
                    _CUDA = _CountingLib(_load("libaxonml_cuda.so", "build_cuda"))
    return _CUDA


def bounds_report():
    """First index violation the debug build recorded since the last call, as a dict, or None.
    Synchronises the device."""
    out = (ctypes.c_int * 6)()
    check(cuda().ax_bounds_read(out), "ax_bounds_read")
    if out[0] == 0:
        return None
    u = lambda lo, hi: (int(lo) & 0xffffffff) | (int(hi) << 32)
    return {"code": int(out[0]), "where": int(out[1]), "index": u(out[2], out[3]), "extent": u(out[4], out[5])}


def launch_count() -> int:
    """Number of native launcher calls made so far in this process."""
    return _CUDA.launches if _CUDA is not None else 0


def host():
    """Handle of the host C++ runtime library."""
    global _HOST
    if _HOST is None:
        with _LOCK:
            if _HOST is None:
                _HOST = _load("libaxonml_host.so", "build_host")
    return _HOST


def have_gpu() -> bool:
    return torch.cuda.is_available()


def is_blackwell() -> bool:
    if not torch.cuda.is_available():
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


def stream_ptr(stream=None) -> c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return c_void_p(s.cuda_stream)


def ptr(t) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


_STATUS = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32[4] status word that kernels write when a bounded wait gives up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index)
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=dev)
        _STATUS[key] = t
    return t


class KernelTimeout(RuntimeError):
    """A bounded device-side wait ran out (the kernel still finished and freed its resources)."""

    def __init__(self, code: int, where: int, block: int):
        super().__init__(f"kernel status code={code} where={where} block={block}")
        self.code, self.where, self.block = code, where, block


def check_status(device=None) -> None:
    """Synchronises and raises ``KernelTimeout`` if any kernel recorded an error."""
    t = status_word(device)
    vals = t.tolist()
    if vals[0] != 0:
        t[:3].zero_()
        raise KernelTimeout(vals[0], vals[1], vals[2])


def set_wait_budget_us(us: int, device=None) -> None:
    """Time budget of every device-side wait (mbarrier, peer signal) of the kernels launched on
    ``device`` from now on, in microseconds; 0 restores the built-in budgets (1 to 2 s).  A wait
    that runs out records code/where/block in the status word and the kernel runs to its end."""
    status_word(device)[3] = int(us)
