"""ONNX import / export (crates/axonml-onnx)."""
from .export import OnnxExporter, export_feedforward, export_module, export_onnx, export_onnx_bytes
from .messages import (ONNX_IR_VERSION, SUPPORTED_OPSET_VERSION, AttributeProto, AttributeType, Dimension, GraphProto, ModelProto,
                       NodeProto, OperatorSetIdProto, StringStringEntry, TensorDataType, TensorProto, TensorShape, TensorType,
                       TypeProto, ValueInfo)
from .model import SUPPORTED_OPS, CompiledOp, ModelInput, OnnxError, OnnxModel, import_onnx, import_onnx_bytes
from .operators import *  # noqa: F401,F403  (OnnxOperator, create_operator and one class per operator)
from .operators import OPERATOR_CLASSES, OnnxOperator, UnsupportedOperator, create_operator

AttributeValue = (int, float, str, list, tuple)      # Python types an exporter attribute may have (export.rs ``AttributeValue``)
