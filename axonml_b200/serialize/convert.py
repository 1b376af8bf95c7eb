"""Key converters between naming schemes (crates/axonml-serialize/src/convert.rs:20-263):
PyTorch <-> AxonML names, ``transpose_linear_weights``, ``OnnxOpType``."""
from __future__ import annotations

import enum

from .state_dict import StateDict, StateDictEntry, TensorData


def convert_from_pytorch_key(key: str) -> str:
    """``module.`` (DataParallel) and ``_orig_mod.`` (compiled) prefixes are dropped; BatchNorm
    bookkeeping keeps its name."""
    for p in ("module.", "_orig_mod."):
        if key.startswith(p):
            key = key[len(p):]
    return key


def convert_to_pytorch_key(key: str) -> str:
    return key


# the reference's function names (convert.rs:20-39)
from_pytorch_key = convert_from_pytorch_key
to_pytorch_key = convert_to_pytorch_key


def convert_from_pytorch(state_dict: StateDict) -> StateDict:
    """A copy of ``state_dict`` with every key passed through ``from_pytorch_key`` (convert.rs:247-256)."""
    out = StateDict()
    for k, e in state_dict.entries():
        out.insert_entry(from_pytorch_key(k), e)
    out.metadata = dict(state_dict.metadata)
    return out


def to_onnx_shape(shape, include_batch: bool = False) -> list:
    """Shape as ONNX dimensions; with ``include_batch`` a dynamic (-1) batch dimension is put in front."""
    dims = [int(d) for d in shape]
    return [-1] + dims if include_batch else dims


def from_onnx_shape(shape, default_dynamic: int = 1) -> list:
    """ONNX dimensions as a concrete shape: dynamic (negative) entries become ``default_dynamic``."""
    return [default_dynamic if int(d) < 0 else int(d) for d in shape]


def from_pytorch_state_dict(tensors: dict) -> StateDict:
    sd = StateDict()
    for k, v in tensors.items():
        if k.endswith("num_batches_tracked"):
            continue
        sd.insert(convert_from_pytorch_key(k), TensorData.from_tensor(v))
    sd.set_metadata("source", "pytorch")
    return sd


def to_pytorch_state_dict(sd: StateDict) -> dict:
    return {convert_to_pytorch_key(k): e.data.to_tensor() for k, e in sd.entries()}


def pytorch_layer_mapping() -> dict:
    return {"Linear": "Linear", "Conv2d": "Conv2d", "BatchNorm2d": "BatchNorm2d", "LayerNorm": "LayerNorm",
            "Embedding": "Embedding", "LSTM": "LSTM", "GRU": "GRU", "MultiheadAttention": "MultiHeadAttention"}


def transpose_linear_weights(sd: StateDict) -> StateDict:
    """Transposes every 2-D ``*.weight`` (for frameworks that store Linear as [in, out])."""
    out = StateDict()
    for k, e in sd.entries():
        if k.endswith("weight") and len(e.data.shape) == 2:
            t = e.data.to_tensor().t().contiguous()
            out.insert_entry(k, StateDictEntry(TensorData.from_tensor(t), e.requires_grad, dict(e.metadata)))
        else:
            out.insert_entry(k, e)
    out.metadata = dict(sd.metadata)
    return out


class OnnxOpType(enum.Enum):
    """ONNX operator names the converters know (convert.rs:93-245)."""
    Add = "Add"
    Sub = "Sub"
    Mul = "Mul"
    Div = "Div"
    MatMul = "MatMul"
    Gemm = "Gemm"
    Relu = "Relu"
    Sigmoid = "Sigmoid"
    Tanh = "Tanh"
    Softmax = "Softmax"
    Gelu = "Gelu"
    Conv = "Conv"
    ConvTranspose = "ConvTranspose"
    MaxPool = "MaxPool"
    AveragePool = "AveragePool"
    GlobalAveragePool = "GlobalAveragePool"
    BatchNormalization = "BatchNormalization"
    LayerNormalization = "LayerNormalization"
    Reshape = "Reshape"
    Transpose = "Transpose"
    Flatten = "Flatten"
    Squeeze = "Squeeze"
    Unsqueeze = "Unsqueeze"
    Concat = "Concat"
    ReduceSum = "ReduceSum"
    ReduceMean = "ReduceMean"
    ReduceMax = "ReduceMax"
    ReduceMin = "ReduceMin"
    Dropout = "Dropout"
    Constant = "Constant"
    Identity = "Identity"
    Unknown = "Unknown"

    @staticmethod
    def from_layer(name: str):
        return {"Linear": OnnxOpType.Gemm, "Conv2d": OnnxOpType.Conv, "ReLU": OnnxOpType.Relu,
                "Sigmoid": OnnxOpType.Sigmoid, "Tanh": OnnxOpType.Tanh, "Softmax": OnnxOpType.Softmax, "GELU": OnnxOpType.Gelu,
                "BatchNorm2d": OnnxOpType.BatchNormalization, "LayerNorm": OnnxOpType.LayerNormalization,
                "MaxPool2d": OnnxOpType.MaxPool, "AvgPool2d": OnnxOpType.AveragePool,
                "AdaptiveAvgPool2d": OnnxOpType.GlobalAveragePool, "Dropout": OnnxOpType.Dropout, "Identity": OnnxOpType.Identity}.get(name)

    @staticmethod
    def from_str(name: str) -> "OnnxOpType":
        """Member with this ONNX name; ``Unknown`` for anything else."""
        try:
            return OnnxOpType(name)
        except ValueError:
            return OnnxOpType.Unknown

    def as_str(self) -> str:
        """The operator's ONNX name."""
        return self.value
