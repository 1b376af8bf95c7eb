"""Core runtime types (crates/axonml-core): Device, DType, errors, storage, backends."""
from .device import (Device, DeviceCapabilities, as_torch_device, cuda_device_count,
                     default_device, vulkan_device_count)
from .dtype import DType, Float, Numeric, Scalar, as_torch_dtype
from .error import *  # noqa: F401,F403
from .error import AxonmlError, Error
from .backends import (BLOCK_SIZE, Backend, BackendType, CpuBackend, CudaBackend, CudaError, CudaKernels, GpuMemory, GpuStream,
                       LaunchConfig,
                       MetalBackend, VulkanBackend, WgpuBackend, best_available_backend, best_available_backend_type, gpu_count,
                       launch_config, stream_synchronize)
from .storage import Allocator, CachingDeviceAllocator, DefaultAllocator, Storage, StorageReadGuard, StorageWriteGuard
