"""Compute backends (crates/axonml-core/src/backends): ``CpuBackend`` = the C++/OpenMP reference
kernels of ``csrc/host/cpu_kernels.cpp`` (static methods on fp32 tensors, cpu.rs:137-731);
``CudaBackend`` = the hand-written sm_100a kernels behind the same method names (the reference's
CUDA island offers add/mul/scale/relu/sigmoid/tanh through sm_50 PTX and cuBLAS sgemm,
cuda.rs:413-629); the graphics-API backends exist as names whose ``is_available()`` is False."""
from __future__ import annotations

import ctypes
import dataclasses
import enum

import torch

from .. import _native as N
from .device import Device
from .error import DeviceNotAvailable as DeviceNotAvailableError

_BIN = {"add": 0, "sub": 1, "mul": 2, "div": 3}
_UN = {"neg": 0, "abs": 1, "relu": 2, "sigmoid": 3, "tanh": 4, "exp": 5, "ln": 6, "sqrt": 7, "square": 8,
       "gelu": 9, "silu": 10, "add_scalar": 11, "mul_scalar": 12, "leaky_relu": 13, "elu": 14}
_RED = {"sum": 0, "prod": 1, "max": 2, "min": 3, "mean": 4, "argmax": 5, "argmin": 6}


def _p(t): return ctypes.c_void_p(t.data_ptr())
def _f(t): return t.detach().to("cpu", torch.float32).contiguous()


class BackendType(enum.Enum):
    """Which kind of device a buffer or stream belongs to (backends/mod.rs:116-132)."""
    Cpu = "cpu"
    Cuda = "cuda"
    Vulkan = "vulkan"
    Metal = "metal"
    Wgpu = "wgpu"


BLOCK_SIZE = 256        # threads per block of the one-dimensional launches (cuda_kernels/mod.rs)


@dataclasses.dataclass(frozen=True)
class LaunchConfig:
    grid_dim: tuple
    block_dim: tuple
    shared_mem_bytes: int = 0


def launch_config(n: int) -> LaunchConfig:
    """One-dimensional launch covering ``n`` elements with 256-thread blocks (cuda_kernels/mod.rs:339-346)."""
    return LaunchConfig(((int(n) + BLOCK_SIZE - 1) // BLOCK_SIZE, 1, 1), (BLOCK_SIZE, 1, 1), 0)


class CudaError(RuntimeError):
    """Failures of the CUDA backend (cuda.rs:272-320), one subclass per variant."""


class DeviceNotFound(CudaError):
    def __init__(self, index=None): super().__init__("CUDA device not found" + (f": {index}" if index is not None else ""))


class CudaAllocationFailed(CudaError):
    def __init__(self, size=None): super().__init__("CUDA memory allocation failed" + (f" ({size} bytes)" if size is not None else ""))


class CopyFailed(CudaError):
    def __init__(self, what=""): super().__init__("CUDA memory copy failed" + (f": {what}" if what else ""))


class KernelLaunchFailed(CudaError):
    def __init__(self, what=""): super().__init__("CUDA kernel launch failed" + (f": {what}" if what else ""))


class BlasError(CudaError):
    def __init__(self, what): super().__init__(f"cuBLAS error: {what}")


class DriverError(CudaError):
    def __init__(self, what): super().__init__(f"CUDA driver error: {what}")


class ModuleLoadFailed(CudaError):
    def __init__(self, what): super().__init__(f"Failed to load CUDA module: {what}")


class KernelNotFound(CudaError):
    def __init__(self, what): super().__init__(f"CUDA kernel not found: {what}")


class GpuMemory:
    """A device allocation by address (backends/mod.rs:108-172).  ``GpuMemory.of(tensor)`` describes
    a tensor's memory and keeps the tensor alive for as long as the handle exists."""

    def __init__(self, ptr: int, size: int, device_index: int, backend_type: BackendType, owner=None):
        self._ptr, self._size, self._device_index, self._backend_type, self._owner = int(ptr), int(size), device_index, backend_type, owner

    @classmethod
    def new(cls, ptr, size, device_index, backend_type): return cls(ptr, size, device_index, backend_type)

    @classmethod
    def of(cls, t: torch.Tensor):
        kind = BackendType.Cuda if t.is_cuda else BackendType.Cpu
        return cls(t.data_ptr(), t.numel() * t.element_size(), t.device.index or 0, kind, t)

    def ptr(self) -> int: return self._ptr
    def size(self) -> int: return self._size
    def device_index(self) -> int: return self._device_index
    def backend_type(self) -> BackendType: return self._backend_type
    def is_null(self) -> bool: return self._ptr == 0
    def __repr__(self) -> str: return f"GpuMemory(0x{self._ptr:x}, {self._size} B, {self._backend_type.value}:{self._device_index})"


def stream_synchronize(handle: int = 0, device_index: int = 0) -> None:
    """Waits for the CUDA stream with this raw handle (0 = the default stream) to drain."""
    if not torch.cuda.is_available():
        return
    if handle == 0:
        torch.cuda.default_stream(device_index).synchronize()
    else:
        torch.cuda.ExternalStream(handle, device=device_index).synchronize()


class GpuStream:
    """A queue of device work by raw handle (backends/mod.rs:176-220)."""

    def __init__(self, handle: int, device_index: int, backend_type: BackendType):
        self._handle, self._device_index, self._backend_type = int(handle), device_index, backend_type

    @classmethod
    def new(cls, handle, device_index, backend_type): return cls(handle, device_index, backend_type)

    @classmethod
    def current(cls, device_index: int = 0):
        """The stream kernels are being launched on right now (a CPU stream when there is no GPU)."""
        if torch.cuda.is_available():
            return cls(torch.cuda.current_stream(device_index).cuda_stream, device_index, BackendType.Cuda)
        return cls(0, 0, BackendType.Cpu)

    def handle(self) -> int: return self._handle
    def device_index(self) -> int: return self._device_index
    def backend_type(self) -> BackendType: return self._backend_type

    def synchronize(self) -> None:
        if self._backend_type is BackendType.Cuda:
            stream_synchronize(self._handle, self._device_index)
        elif self._backend_type is not BackendType.Cpu:
            raise DeviceNotAvailableError(self._backend_type.value)


# module-level queries of the CUDA backend (crates/axonml-core/src/backends/cuda.rs ``is_available``,
# ``device_count``, ``is_device_available``, ``get_capabilities``)
def is_available() -> bool:
    return torch.cuda.is_available()


def device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def is_device_available(index: int) -> bool:
    return 0 <= index < device_count()


def get_capabilities(index: int = 0):
    """``DeviceCapabilities`` of CUDA device ``index``; raises ``DeviceNotFound`` when there is none."""
    if not is_device_available(index):
        raise DeviceNotFound(index)
    return Device.Cuda(index).capabilities()


class CudaKernels:
    """The kernel library as an object (backends/cuda_kernels/mod.rs ``CudaKernels``: the loaded
    module plus launch helpers).  The reference embeds PTX for six elementwise kernels; here the
    object fronts the sm_100a library the package is built with: ``has(name)`` says whether an
    entry point exists, ``launch_elementwise`` runs one of the unary / binary elementwise kernels."""
    @property
    def UNARY(self) -> tuple:
        from ..ops import elementwise
        return tuple(elementwise.UNARY)

    @property
    def BINARY(self) -> tuple:
        from ..ops import elementwise
        return tuple(elementwise.BINARY)

    def __init__(self, device_index: int = 0):
        if not is_device_available(device_index):
            raise DeviceNotFound(device_index)
        self.device_index = device_index
        try:
            self._lib = N.cuda()
        except Exception as e:  # noqa: BLE001 - any loader failure is a module-load failure here
            raise ModuleLoadFailed(str(e)) from e

    @classmethod
    def load(cls, device_index: int = 0): return cls(device_index)

    def has(self, entry_point: str) -> bool:
        return hasattr(getattr(self._lib, "_lib", self._lib), entry_point)        # dlsym through ctypes

    def launch_config(self, n: int) -> LaunchConfig:
        return launch_config(n)

    def get(self, entry_point: str):
        """The library's callable for ``entry_point``; ``KernelNotFound`` when it has none (mod.rs ``get``)."""
        if not self.has(entry_point):
            raise KernelNotFound(entry_point)
        return getattr(self._lib, entry_point)

    def launch_elementwise(self, name: str, *tensors, alpha: float = 0.0):
        from ..ops import elementwise
        if name in self.BINARY and len(tensors) == 2:
            return elementwise.binary(tensors[0], tensors[1], name)
        if name in self.UNARY and len(tensors) == 1:
            return elementwise.unary(tensors[0], name, alpha)
        raise KernelNotFound(f"{name} with {len(tensors)} operands")


def gpu_count() -> int:
    """Devices over all GPU backends (backends/mod.rs:266-291): the CUDA devices here."""
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def best_available_backend_type() -> BackendType:
    return BackendType.Cuda if torch.cuda.is_available() else BackendType.Cpu


class Backend:
    """alloc / copy / sync surface of the reference's ``Backend`` trait (backends/mod.rs:73-100)."""
    def name(self) -> str: raise NotImplementedError
    def is_available(self) -> bool: return False
    def device(self) -> Device: raise NotImplementedError
    def allocate(self, count: int, dtype=torch.float32): return torch.empty(count, dtype=dtype, device=self.device().to_torch())
    def copy_to_device(self, host: torch.Tensor): return host.to(self.device().to_torch())
    def copy_to_host(self, dev: torch.Tensor): return dev.cpu()
    def synchronize(self) -> None: pass


class CpuBackend(Backend):
    def name(self) -> str: return "cpu"
    def backend_type(self) -> BackendType: return BackendType.Cpu
    def is_available(self) -> bool: return True
    def device(self) -> Device: return Device.Cpu()

    @staticmethod
    def _binary(op, a, b):
        a, b = _f(a), _f(b)
        y = torch.empty_like(a)
        N.host().ax_cpu_binary(_BIN[op], _p(a), _p(b), _p(y), ctypes.c_int64(a.numel()))
        return y

    @staticmethod
    def _unary(op, x, p=0.0):
        x = _f(x)
        y = torch.empty_like(x)
        N.host().ax_cpu_unary(_UN[op], _p(x), _p(y), ctypes.c_int64(x.numel()), ctypes.c_float(p))
        return y

    @staticmethod
    def _reduce(op, x):
        x = _f(x)
        fn = N.host().ax_cpu_reduce
        fn.restype = ctypes.c_double
        return fn(_RED[op], _p(x), ctypes.c_int64(x.numel()))

    add = staticmethod(lambda a, b: CpuBackend._binary("add", a, b))
    sub = staticmethod(lambda a, b: CpuBackend._binary("sub", a, b))
    mul = staticmethod(lambda a, b: CpuBackend._binary("mul", a, b))
    div = staticmethod(lambda a, b: CpuBackend._binary("div", a, b))
    add_scalar = staticmethod(lambda x, s: CpuBackend._unary("add_scalar", x, s))
    mul_scalar = staticmethod(lambda x, s: CpuBackend._unary("mul_scalar", x, s))
    neg = staticmethod(lambda x: CpuBackend._unary("neg", x))
    abs = staticmethod(lambda x: CpuBackend._unary("abs", x))
    relu = staticmethod(lambda x: CpuBackend._unary("relu", x))
    sigmoid = staticmethod(lambda x: CpuBackend._unary("sigmoid", x))
    tanh = staticmethod(lambda x: CpuBackend._unary("tanh", x))
    exp = staticmethod(lambda x: CpuBackend._unary("exp", x))
    ln = staticmethod(lambda x: CpuBackend._unary("ln", x))
    sqrt = staticmethod(lambda x: CpuBackend._unary("sqrt", x))
    square = staticmethod(lambda x: CpuBackend._unary("square", x))
    gelu = staticmethod(lambda x: CpuBackend._unary("gelu", x))
    silu = staticmethod(lambda x: CpuBackend._unary("silu", x))
    sum = staticmethod(lambda x: CpuBackend._reduce("sum", x))
    prod = staticmethod(lambda x: CpuBackend._reduce("prod", x))
    max = staticmethod(lambda x: CpuBackend._reduce("max", x))
    min = staticmethod(lambda x: CpuBackend._reduce("min", x))
    mean = staticmethod(lambda x: CpuBackend._reduce("mean", x))
    argmax = staticmethod(lambda x: int(CpuBackend._reduce("argmax", x)))
    argmin = staticmethod(lambda x: int(CpuBackend._reduce("argmin", x)))

    @staticmethod
    def matmul(a, b):
        a, b = _f(a), _f(b)
        M, K = a.shape
        K2, Nn = b.shape
        c = torch.empty(M, Nn)
        N.host().ax_cpu_matmul(_p(a), _p(b), _p(c), ctypes.c_int64(M), ctypes.c_int64(Nn), ctypes.c_int64(K))
        return c

    @staticmethod
    def sgemm(c, a, b, m: int, n: int, k: int, alpha: float = 1.0, beta: float = 0.0):
        """C[m, n] = alpha * A[m, k] B[k, n] + beta * C, in place on the fp32 tensor ``c`` (cpu.rs:566-600)."""
        prod = CpuBackend.matmul(a.reshape(m, k), b.reshape(k, n))
        out = c.view(m, n)
        out.copy_(alpha * prod + (beta * out if beta != 0.0 else 0.0))
        return c

    @staticmethod
    def dgemm(c, a, b, m: int, n: int, k: int, alpha: float = 1.0, beta: float = 0.0):
        """The fp64 form of ``sgemm`` (cpu.rs:603-636)."""
        prod = a.reshape(m, k).double() @ b.reshape(k, n).double()
        out = c.view(m, n)
        out.copy_(alpha * prod + (beta * out if beta != 0.0 else 0.0))
        return c

    @staticmethod
    def matmul_f32(c, a, b, m: int, n: int, k: int): return CpuBackend.sgemm(c, a, b, m, n, k, 1.0, 0.0)
    @staticmethod
    def matmul_f64(c, a, b, m: int, n: int, k: int): return CpuBackend.dgemm(c, a, b, m, n, k, 1.0, 0.0)

    @staticmethod
    def fill(dst, value):
        dst.fill_(value)
        return dst

    @staticmethod
    def fill_zeros(dst): return CpuBackend.fill(dst, 0)

    @staticmethod
    def copy(dst, src):
        if dst.numel() != src.numel():
            raise ValueError(f"copy of {src.numel()} elements into {dst.numel()}")
        dst.view(-1).copy_(src.reshape(-1))
        return dst

    @staticmethod
    def transpose(x):
        x = _f(x)
        y = torch.empty(x.shape[1], x.shape[0])
        N.host().ax_cpu_transpose(_p(x), _p(y), ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]))
        return y

    @staticmethod
    def dot(a, b):
        a, b = _f(a), _f(b)
        fn = N.host().ax_cpu_dot
        fn.restype = ctypes.c_double
        return fn(_p(a), _p(b), ctypes.c_int64(a.numel()))

    @staticmethod
    def _cmp(op, a, b):
        a, b = _f(a), _f(b)
        y = torch.empty_like(a)
        N.host().ax_cpu_compare(op, _p(a), _p(b), _p(y), ctypes.c_int64(a.numel()))
        return y

    eq = staticmethod(lambda a, b: CpuBackend._cmp(0, a, b))
    lt = staticmethod(lambda a, b: CpuBackend._cmp(1, a, b))
    gt = staticmethod(lambda a, b: CpuBackend._cmp(2, a, b))

    @staticmethod
    def conv2d(x, w, bias=None, stride=1, padding=0):
        x, w = _f(x), _f(w)
        Nb, C, H, W = x.shape
        O, _, KH, KW = w.shape
        OH, OW = (H + 2 * padding - KH) // stride + 1, (W + 2 * padding - KW) // stride + 1
        y = torch.empty(Nb, O, OH, OW)
        b = _f(bias) if bias is not None else None
        N.host().ax_cpu_conv2d(_p(x), _p(w), _p(b) if b is not None else ctypes.c_void_p(0), _p(y), Nb, C, H, W, O, KH, KW,
                               stride, stride, padding, padding)
        return y

    @staticmethod
    def softmax_rows(x, log: bool = False):
        x = _f(x)
        y = torch.empty_like(x)
        N.host().ax_cpu_softmax_rows(_p(x), _p(y), ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]), int(log))
        return y

    @staticmethod
    def layer_norm(x, w=None, b=None, eps=1e-5, rms=False):
        x = _f(x)
        y = torch.empty_like(x)
        wf, bf = (_f(w) if w is not None else None), (_f(b) if b is not None else None)
        N.host().ax_cpu_layer_norm(_p(x), _p(wf) if wf is not None else ctypes.c_void_p(0),
                                   _p(bf) if bf is not None else ctypes.c_void_p(0), _p(y),
                                   ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]), ctypes.c_float(eps), int(rms))
        return y

    @staticmethod
    def flash_attention(q, k, v, causal=False, scale=None, block=64):
        q, k, v = _f(q), _f(k), _f(v)
        BH, Sq, D = q.shape
        o = torch.empty_like(q)
        N.host().ax_cpu_flash_attention(_p(q), _p(k), _p(v), _p(o), BH, Sq, k.shape[1], D,
                                        ctypes.c_float(scale if scale is not None else D ** -0.5), int(causal), block)
        return o


class CudaBackend(Backend):
    def __init__(self, index: int = 0): self.index = index
    def name(self) -> str: return "cuda"
    def backend_type(self) -> BackendType: return BackendType.Cuda
    def is_available(self) -> bool: return torch.cuda.is_available() and self.index < torch.cuda.device_count()
    def device(self) -> Device: return Device.Cuda(self.index)
    def synchronize(self) -> None: torch.cuda.synchronize(self.index)
    def stream_synchronize(self) -> None: torch.cuda.current_stream(self.index).synchronize()
    def mem_get_info(self): return torch.cuda.mem_get_info(self.index)
    def device_index(self) -> int: return self.index

    def blas(self):
        """Handle of the library GEMM context of this device (the reference exposes its cuBLAS
        handle); plain library GEMMs here go through torch, so this is torch's handle."""
        with torch.cuda.device(self.index):
            return torch.cuda.current_blas_handle()

    def alloc(self, count: int, dtype=torch.float32) -> torch.Tensor:
        """``count`` zeroed elements on the device (cuda.rs ``alloc``)."""
        return torch.zeros(count, dtype=dtype, device=f"cuda:{self.index}")

    def alloc_uninit(self, count: int, dtype=torch.float32) -> torch.Tensor:
        return torch.empty(count, dtype=dtype, device=f"cuda:{self.index}")

    def htod_copy(self, host, non_blocking: bool = False) -> torch.Tensor:
        """Host data (tensor, list or array) -> a new device tensor."""
        return torch.as_tensor(host).to(f"cuda:{self.index}", non_blocking=non_blocking)

    def dtoh_copy(self, dev: torch.Tensor) -> torch.Tensor:
        return dev.detach().cpu()

    def _e(self):
        from ..ops import elementwise
        return elementwise

    def add_f32(self, a, b): return self._e().binary(a, b, "add")
    def sub_f32(self, a, b): return self._e().binary(a, b, "sub")
    def mul_f32(self, a, b): return self._e().binary(a, b, "mul")
    def div_f32(self, a, b): return self._e().binary(a, b, "div")
    def scale_f32(self, x, alpha): return self._e().unary(x, "scale", alpha, out=x)
    def relu_f32(self, x): return self._e().unary(x, "relu")
    def sigmoid_f32(self, x): return self._e().unary(x, "sigmoid")
    def tanh_f32(self, x): return self._e().unary(x, "tanh")
    def gelu_f32(self, x): return self._e().unary(x, "gelu")
    def silu_f32(self, x): return self._e().unary(x, "silu")

    def gemm_f32(self, a, b):
        """C = A B in fp32 (fp32 multiply-add and accumulation on the CUDA cores, the precision of the
        reference's cuBLAS sgemm; tolerance of its GEMM test: 1e-3 / 1e-2)."""
        from ..ops.gemm import sgemm_f32
        return sgemm_f32(a.float(), b.float())

    def gemm_batched_f32(self, a, b):
        """Batched C[i] = A[i] B[i] in one launch (cuda.rs:454-501, sgemmStridedBatched)."""
        from ..ops.gemm import sgemm_f32
        a = torch.stack(list(a)) if not torch.is_tensor(a) else a
        b = torch.stack(list(b)) if not torch.is_tensor(b) else b
        return sgemm_f32(a.float(), b.float())


class _Unavailable(Backend):
    NAME = "none"
    def name(self) -> str: return self.NAME
    def backend_type(self) -> BackendType: return BackendType(self.NAME)
    def is_available(self) -> bool: return False
    def device(self) -> Device: return Device(self.NAME, 0)


class VulkanBackend(_Unavailable): NAME = "vulkan"
class MetalBackend(_Unavailable): NAME = "metal"
class WgpuBackend(_Unavailable): NAME = "wgpu"


def best_available_backend() -> Backend:
    return CudaBackend(torch.cuda.current_device()) if torch.cuda.is_available() else CpuBackend()
