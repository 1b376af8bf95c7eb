"""Registry of pretrained vision models, their weight cache and the hub's weight file format.

Parity: crates/axonml-vision/src/hub.rs (``PretrainedModel{name, url, checksum, size_bytes,
num_classes, input_size, dataset, accuracy}``, ``model_registry`` with the ResNet, VGG, MobileNet,
EfficientNet, DenseNet, ViT, Swin and ConvNeXt entries, ``cache_dir`` = ``<cache>/axonml/hub/
weights``, ``is_cached`` / ``cached_path``, ``download_weights(name, force)``, ``save_state_dict`` /
``load_state_dict`` in the hub's binary format ``u32 n; n x {u32 name_len, name, u32 ndim, ndim x
u64, f32 data}`` (:514-596), ``list_models``, ``model_info``).  Sizes and ImageNet-1K top-1
accuracies are the published figures of each architecture."""
from __future__ import annotations

import dataclasses
import os

from ..hub import load_hub_weights, save_hub_weights
from ..hub.download import HubError, InvalidFormat, ModelNotFound, fetch, hub_cache_root, repo_url  # noqa: F401


@dataclasses.dataclass(frozen=True)
class PretrainedModel:
    name: str
    size_bytes: int
    accuracy: float                   # ImageNet-1K top-1, per cent
    num_classes: int = 1000
    input_size: tuple = (224, 224)
    dataset: str = "ImageNet-1K"
    checksum: str | None = None

    @property
    def repo(self) -> str:
        return f"axonml-ml/{self.name.replace('_', '-')}-imagenet"

    @property
    def url(self) -> str:
        return repo_url(self.repo, self.name + ".safetensors")


def _e(name, mb, acc, input_size=(224, 224)):
    return PretrainedModel(name, int(mb * 1_000_000), acc, input_size=input_size)


_ENTRIES = [
    _e("resnet18", 44.7, 69.76), _e("resnet34", 83.3, 73.31), _e("resnet50", 97.8, 76.13), _e("resnet101", 170.5, 77.37),
    _e("resnet152", 230.4, 78.31),
    _e("vgg16", 527.8, 71.59), _e("vgg19", 548.1, 72.38), _e("vgg16_bn", 527.9, 73.36),
    _e("mobilenet_v2", 13.6, 71.88), _e("mobilenet_v3_small", 9.8, 67.67), _e("mobilenet_v3_large", 21.1, 74.04),
    _e("efficientnet_b0", 20.5, 77.69), _e("efficientnet_b1", 30.1, 78.64, (240, 240)), _e("efficientnet_b2", 35.2, 80.61, (260, 260)),
    _e("densenet121", 30.8, 74.43), _e("densenet169", 54.7, 75.60),
    _e("vit_b_16", 330.3, 81.07), _e("vit_b_32", 336.6, 75.91),
    _e("swin_t", 108.2, 81.47), _e("swin_s", 189.8, 83.20),
    _e("convnext_tiny", 109.1, 82.52), _e("convnext_small", 191.7, 83.62),
]


def model_registry() -> dict:
    return {m.name: m for m in _ENTRIES}


def cache_dir() -> str:
    return os.path.join(hub_cache_root(), "weights")


def cached_path(model_name: str) -> str:
    return os.path.join(cache_dir(), model_name + ".safetensors")


def is_cached(model_name: str) -> bool:
    return os.path.exists(cached_path(model_name))


def download_weights(model_name: str, force: bool = False, quiet: bool = False) -> str:
    info = model_registry().get(model_name)
    if info is None:
        raise ModelNotFound(model_name)
    path = cached_path(model_name)
    if os.path.exists(path) and not force:
        return path
    if not quiet:
        print(f"Downloading {model_name} weights ({info.size_bytes / 1e6:.1f} MB)...")
    fetch(info.url, path, info.checksum)
    if not quiet:
        print(f"Downloaded to {path}")
    return path


def save_state_dict(state: dict, path: str) -> None:
    """Writes ``{name: tensor}`` in the hub's binary format (fp32 data)."""
    save_hub_weights(state, path)


def load_state_dict(path: str) -> dict:
    """Reads a file written by ``save_state_dict``; SafeTensors files are recognised as well."""
    import struct
    with open(path, "rb") as f:
        head = f.read(16)
    if len(head) >= 9 and head[8:9] == b"{":                    # u64 header length, then JSON
        from ..serialize.codec import safetensors_loads
        with open(path, "rb") as f:
            return safetensors_loads(f.read())[0]
    try:
        return load_hub_weights(path)
    except (struct.error, UnicodeDecodeError, ValueError) as e:
        raise InvalidFormat(f"{path}: {e}") from e


def list_models() -> list:
    return list(_ENTRIES)


def model_info(name: str):
    return model_registry().get(name)
