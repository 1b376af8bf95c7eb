"""Device handle.  Mirrors ``Device`` and ``DeviceCapabilities`` of
crates/axonml-core/src/device.rs:38-58, :157-236.  Only ``Cpu`` and ``Cuda(i)`` can hold data
in this build; the graphics-API variants exist as names and always report unavailable."""
from __future__ import annotations

import dataclasses
import os

import torch


@dataclasses.dataclass(frozen=True)
class DeviceCapabilities:
    name: str
    supports_f64: bool
    supports_f16: bool
    supports_bf16: bool
    total_memory: int
    available_memory: int
    max_threads_per_block: int
    compute_capability: tuple | None
    sm_count: int = 0


@dataclasses.dataclass(frozen=True)
class Device:
    kind: str = "cpu"
    index: int = 0

    # ---- constructors named after the reference's variants
    @staticmethod
    def Cpu() -> "Device":
        return Device("cpu", 0)

    @staticmethod
    def Cuda(index: int = 0) -> "Device":
        return Device("cuda", index)

    @staticmethod
    def Vulkan(index: int = 0) -> "Device":
        return Device("vulkan", index)

    @staticmethod
    def Metal(index: int = 0) -> "Device":
        return Device("metal", index)

    @staticmethod
    def Wgpu(index: int = 0) -> "Device":
        return Device("wgpu", index)

    @staticmethod
    def parse(text: str) -> "Device":
        text = text.strip().lower()
        if text in ("cpu", ""):
            return Device.Cpu()
        kind, _, idx = text.partition(":")
        if kind == "gpu":
            kind = "cuda"
        return Device(kind, int(idx) if idx else 0)

    @staticmethod
    def from_torch(dev) -> "Device":
        dev = torch.device(dev)
        return Device(dev.type, dev.index or 0)

    # ---- reference API
    def is_available(self) -> bool:
        if self.kind == "cpu":
            return True
        if self.kind == "cuda":
            return torch.cuda.is_available() and self.index < torch.cuda.device_count()
        return False  # graphics-API devices cannot be brought up here

    def is_cpu(self) -> bool:
        return self.kind == "cpu"

    def is_gpu(self) -> bool:
        return self.kind != "cpu"

    def device_index(self) -> int:
        return self.index

    def device_name(self) -> str:
        if self.kind == "cuda" and self.is_available():
            return torch.cuda.get_device_name(self.index)
        return str(self)

    def capabilities(self) -> DeviceCapabilities:
        if self.kind == "cuda" and self.is_available():
            p = torch.cuda.get_device_properties(self.index)
            free, total = torch.cuda.mem_get_info(self.index)
            return DeviceCapabilities(p.name, True, True, p.major >= 8, total, free,
                                      p.max_threads_per_multi_processor and 1024,
                                      (p.major, p.minor), p.multi_processor_count)
        try:
            import psutil
            vm = psutil.virtual_memory()
            total, avail = vm.total, vm.available
        except Exception:  # pragma: no cover
            total = avail = 0
        return DeviceCapabilities("CPU", True, True, True, total, avail, os.cpu_count() or 1, None)

    def to_torch(self) -> torch.device:
        if self.kind == "cpu":
            return torch.device("cpu")
        if self.kind == "cuda":
            return torch.device("cuda", self.index)
        from .error import DeviceNotAvailable
        raise DeviceNotAvailable(str(self))

    def __str__(self) -> str:
        return "cpu" if self.kind == "cpu" else f"{self.kind}:{self.index}"


def cuda_device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def vulkan_device_count() -> int:
    return 0


def as_torch_device(dev) -> torch.device:
    if isinstance(dev, Device):
        return dev.to_torch()
    return torch.device(dev)


def default_device() -> Device:
    return Device.Cuda(torch.cuda.current_device()) if torch.cuda.is_available() else Device.Cpu()
