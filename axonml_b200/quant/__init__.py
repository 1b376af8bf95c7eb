"""Quantisation (crates/axonml-quant) and the GGUF container."""
from .calibration import CalibrationData, CalibrationMethod, calibrate, calibrate_batch
from .gguf import GGUFFile, read_gguf, write_gguf
from .quantize import (QuantizationStats, compute_quantization_error, compute_quantization_stats,
                       dequantize_block, dequantize_tensor, quantize_model, quantize_tensor)
from .types import (DEFAULT_BLOCK_SIZE, MAX_BLOCK_SIZE, Q4_1Block, Q4Block, Q8Block, QuantError, QuantizedBlock, QuantizedTensor,
                    QuantType)
