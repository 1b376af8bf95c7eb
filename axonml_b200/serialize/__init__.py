"""Checkpoint containers and codecs (crates/axonml-serialize): ``save_model``,
``save_state_dict``, ``load_state_dict``, ``save_checkpoint``, ``load_checkpoint`` pick the codec
from the file extension (``.axonml``/``.bin`` bincode, ``.json``, ``.safetensors``/``.st``,
``.gguf``)."""
from __future__ import annotations

import os

from . import codec
from .checkpoint import (Checkpoint, CheckpointBuilder, TrainingState, decode_checkpoint,
                         encode_checkpoint, optimizer_from_state_dict, optimizer_to_state_dict)
from .convert import (OnnxOpType, convert_from_pytorch, convert_from_pytorch_key, convert_to_pytorch_key, from_onnx_shape,
                      from_pytorch_key, from_pytorch_state_dict, pytorch_layer_mapping, to_onnx_shape, to_pytorch_key,
                      to_pytorch_state_dict, transpose_linear_weights)
from .format import Format, detect_format, detect_format_from_bytes
from .state_dict import StateDict, StateDictEntry, TensorData


def save_state_dict(sd: StateDict, path, fmt: Format | None = None) -> None:
    fmt = fmt or detect_format(path)
    if fmt is Format.Axonml:
        data = codec.encode_state_dict(sd)
    elif fmt is Format.Json:
        data = codec.state_dict_to_json(sd).encode()
    elif fmt is Format.SafeTensors:
        data = codec.safetensors_dumps(sd.to_tensors(), sd.metadata)
    elif fmt is Format.Gguf:
        from ..quant import gguf
        gguf.write_gguf(path, sd.to_tensors(), {"general.name": sd.metadata.get("name", "axonml")})
        return
    else:  # pragma: no cover
        raise ValueError(fmt)
    tmp = str(path) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(data)
    os.replace(tmp, path)


def load_state_dict(path, fmt: Format | None = None) -> StateDict:
    with open(path, "rb") as f:
        data = f.read()
    fmt = fmt or detect_format(path)
    if fmt is Format.Axonml:
        return codec.decode_state_dict(data)[0]
    if fmt is Format.Json:
        return codec.state_dict_from_json(data.decode())
    if fmt is Format.SafeTensors:
        tensors, meta = codec.safetensors_loads(data)
        sd = StateDict.from_tensors({k: v.float() for k, v in tensors.items()})
        sd.metadata = {k: v for k, v in meta.items() if not k.endswith(".shape")}
        return sd
    if fmt is Format.Gguf:
        from ..quant import gguf
        g = gguf.read_gguf(path)
        return StateDict.from_tensors({k: g.tensor(k).float() for k in g.tensor_names()})
    raise ValueError(fmt)


def save_model(module, path, fmt: Format | None = None) -> None:
    save_state_dict(StateDict.from_module(module), path, fmt)


def load_model(module, path, strict: bool = True):
    return load_state_dict(path).load_into(module, strict)


def save_checkpoint(ck: Checkpoint, path) -> None:
    tmp = str(path) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(encode_checkpoint(ck))
    os.replace(tmp, path)


def load_checkpoint(path) -> Checkpoint:
    with open(path, "rb") as f:
        return decode_checkpoint(f.read())
