"""ONNX import / export (crates/axonml-onnx)."""
from .export import OnnxExporter, export_feedforward, export_module, export_onnx, export_onnx_bytes
from .model import SUPPORTED_OPS, CompiledOp, ModelInput, OnnxError, OnnxModel, import_onnx, import_onnx_bytes
