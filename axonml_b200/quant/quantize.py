"""Quantise / dequantise tensors and models (crates/axonml-quant/src/quantize.rs:36-290,
dequantize.rs:20-125).  CPU tensors go through the C++ codecs (``csrc/host/quant.cpp``), CUDA
tensors through the block-quantise kernels (``csrc/kernels/quant.cu``); both produce GGML layouts,
so a tensor quantised on the GPU can be written to a GGUF file directly."""
from __future__ import annotations

import ctypes
import dataclasses

import torch

from .. import _native as N
from .types import QuantError, QuantizedTensor, QuantType


def _pad_rows(t: torch.Tensor, block: int) -> torch.Tensor:
    if t.shape[-1] % block == 0:
        return t
    raise QuantError(f"last dimension {t.shape[-1]} is not a multiple of the block size {block}")


def quantize_tensor(t: torch.Tensor, quant_type: QuantType, layout: str = "ggml") -> QuantizedTensor:
    if not quant_type.is_block_quantized():
        dt = {QuantType.F16: torch.float16, QuantType.BF16: torch.bfloat16, QuantType.F32: torch.float32}[quant_type]
        return QuantizedTensor(list(t.shape), quant_type, t.detach().to(dt).contiguous().view(-1).view(torch.uint8), layout)
    block = quant_type.block_size()
    flat = t.detach()
    if flat.numel() % block:
        raise QuantError(f"{flat.numel()} elements are not a multiple of the block size {block}")
    nb = flat.numel() // block
    if flat.is_cuda and N.have_gpu() and layout == "ggml":
        from ..ops import quant as Q
        return QuantizedTensor(list(t.shape), quant_type, Q.quantize_cuda(flat, quant_type), layout)
    x = flat.to("cpu", torch.float32).contiguous().view(-1)
    out = torch.empty(nb * quant_type.bytes_per_block(), dtype=torch.uint8)
    rc = N.host().ax_quantize(quant_type.codec_id(), 1 if layout == "adjacent" else 0,
                              ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                              ctypes.c_int64(x.numel()))
    if rc != 0:
        raise QuantError("quantisation failed")
    return QuantizedTensor(list(t.shape), quant_type, out.to(t.device) if t.is_cuda else out, layout)


def dequantize_tensor(q: QuantizedTensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    qt = q.quant_type
    if not qt.is_block_quantized():
        dt = {QuantType.F16: torch.float16, QuantType.BF16: torch.bfloat16, QuantType.F32: torch.float32}[qt]
        return q.data.view(dt).view(q.shape).to(dtype)
    if q.data.is_cuda and N.have_gpu() and q.layout == "ggml":
        from ..ops import quant as Q
        return Q.dequantize_cuda(q.data, qt, q.numel(), dtype).view(q.shape)
    data = q.data.cpu().contiguous()
    y = torch.empty(q.numel(), dtype=torch.float32)
    rc = N.host().ax_dequantize(qt.codec_id(), 1 if q.layout == "adjacent" else 0,
                                ctypes.c_void_p(data.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                ctypes.c_int64(q.numel()))
    if rc != 0:
        raise QuantError("dequantisation failed")
    return y.view(q.shape).to(dtype)


def dequantize_block(block_bytes: bytes, quant_type: QuantType) -> list:
    q = QuantizedTensor([quant_type.block_size()], quant_type, torch.frombuffer(bytearray(block_bytes), dtype=torch.uint8))
    return dequantize_tensor(q).tolist()


def quantize_model(named_tensors, quant_type: QuantType, min_numel: int = 1024) -> dict:
    """Quantises every (name, tensor) whose element count is a multiple of the block size and at
    least ``min_numel``; the rest stay in fp32 (quantize.rs:64-80)."""
    out = {}
    items = named_tensors.items() if isinstance(named_tensors, dict) else named_tensors
    for name, t in items:
        if t.numel() >= min_numel and t.numel() % quant_type.block_size() == 0 and t.dim() >= 2:
            out[name] = quantize_tensor(t, quant_type)
        else:
            out[name] = quantize_tensor(t, QuantType.F32)
    return out


def compute_quantization_error(original, dequantized) -> float:
    """Root-mean-square error (quantize.rs:235-249)."""
    a, b = torch.as_tensor(original, dtype=torch.float32), torch.as_tensor(dequantized, dtype=torch.float32)
    return float(((a - b) ** 2).mean().sqrt())


@dataclasses.dataclass
class QuantizationStats:
    rmse: float
    max_error: float
    mean_error: float
    compression_ratio: float


def compute_quantization_stats(original: torch.Tensor, dequantized: torch.Tensor, quant_type: QuantType):
    d = (original.float() - dequantized.float()).abs()
    return QuantizationStats(float((d ** 2).mean().sqrt()), float(d.max()), float(d.mean()),
                             quant_type.compression_ratio())
