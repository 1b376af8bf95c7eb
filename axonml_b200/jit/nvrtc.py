"""Run-time compilation of generated CUDA C with NVRTC for sm_100a and launch through the driver
API (cuda-python bindings).  Used by the JIT and fusion code generators; no Triton, no
torch.compile."""
from __future__ import annotations

import ctypes

import torch

from .error import CompilationFailed, JitRuntimeError


def _bindings():
    try:
        from cuda.bindings import driver, nvrtc
    except Exception:
        from cuda import cuda as driver, nvrtc          # older cuda-python layout
    return driver, nvrtc


def available() -> bool:
    if not torch.cuda.is_available():
        return False
    try:
        _bindings()
        return True
    except Exception:
        return False


class Module:
    """One NVRTC compilation unit loaded into the current context; ``function(name)`` returns a
    launchable entry point."""

    def __init__(self, source: str):
        driver, nvrtc = _bindings()
        self._driver = driver
        err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b"axonml_jit.cu", 0, [], [])
        major, minor = torch.cuda.get_device_capability()
        arch = f"sm_{major}{minor}a" if major >= 9 else f"sm_{major}{minor}"
        opts = [f"--gpu-architecture={arch}".encode(), b"--use_fast_math", b"-default-device"]
        (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
        if int(err) != 0:
            _, n = nvrtc.nvrtcGetProgramLogSize(prog)
            log = b" " * n
            nvrtc.nvrtcGetProgramLog(prog, log)
            raise CompilationFailed("NVRTC:\n" + log.decode(errors="replace") + "\n" + source)
        _, n = nvrtc.nvrtcGetCUBINSize(prog)
        cubin = b" " * n
        nvrtc.nvrtcGetCUBIN(prog, cubin)
        torch.cuda.init()
        torch.zeros(1, device="cuda")          # make sure the primary context is current
        err, self._module = driver.cuModuleLoadData(cubin)
        if int(err) != 0:
            raise CompilationFailed(f"cuModuleLoadData: {err}")
        self.source = source

    def function(self, name: str) -> "Function":
        err, fn = self._driver.cuModuleGetFunction(self._module, name.encode())
        if int(err) != 0:
            raise CompilationFailed(f"cuModuleGetFunction({name}): {err}")
        return Function(self, fn)


class Function:
    def __init__(self, module: Module, fn):
        self._module, self._fn = module, fn      # the module must outlive its functions

    def launch(self, grid: int, block: int, args, arg_types) -> None:
        """``args``: python ints (device pointers, sizes) / floats; ``arg_types``: ctypes types."""
        driver = self._module._driver
        stream = torch.cuda.current_stream().cuda_stream
        (err,) = driver.cuLaunchKernel(self._fn, grid, 1, 1, block, 1, 1, 0, stream, (tuple(args), tuple(arg_types)), 0)
        if int(err) != 0:
            raise JitRuntimeError(f"cuLaunchKernel: {err}")


class Kernel(Function):
    """A module with a single entry point."""

    def __init__(self, source: str, name: str):
        mod = Module(source)
        f = mod.function(name)
        super().__init__(mod, f._fn)
        self.source = source
