"""Quantisation (crates/axonml-quant) and the GGUF container."""
from .calibration import CalibrationData, CalibrationMethod, calibrate, calibrate_batch
from .gguf import GGUFFile, read_gguf, write_gguf
from .quantize import (QuantizationStats, compute_quantization_error, compute_quantization_stats,
                       dequantize_block, dequantize_tensor, quantize_model, quantize_tensor)
from .types import QuantError, QuantizedBlock, QuantizedTensor, QuantType
