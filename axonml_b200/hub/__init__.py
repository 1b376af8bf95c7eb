"""Model hubs (crates/axonml/src/hub.rs:32-414, crates/axonml-vision/src/hub.rs:74-603,
crates/axonml-llm/src/hub.rs): a unified registry of the models this package can build, search /
filter helpers, ``BenchmarkResult``, a local weight cache, and the vision hub's own binary weight
format ``u32 n; repeat{u32 name_len, name, u32 ndim, ndim x u64 dims, f32 data}``
(vision/hub.rs:514-596)."""
from __future__ import annotations

import dataclasses
import enum
import os
import struct

import numpy as np
import torch

from ..benchmark import BenchmarkResult, compare_benchmarks  # noqa: F401


class ModelCategory(enum.Enum):
    Vision = "vision"
    Language = "language"
    Audio = "audio"
    Multimodal = "multimodal"


@dataclasses.dataclass
class UnifiedModelInfo:
    name: str
    category: ModelCategory
    architecture: str
    num_parameters: int
    size_bytes: int
    description: str
    tasks: tuple
    builder: object = None

    def size_mb(self) -> float: return self.size_bytes / 2 ** 20

    def params_str(self) -> str:
        n = self.num_parameters
        return f"{n / 1e9:.1f}B" if n >= 1e9 else f"{n / 1e6:.1f}M" if n >= 1e6 else f"{n / 1e3:.1f}K"

    def build(self, **kw):
        return self.builder(**kw)


def _v(name, arch, params, desc, tasks, builder):
    return UnifiedModelInfo(name, ModelCategory.Vision, arch, params, params * 4, desc, tasks, builder)


def _l(name, arch, params, desc, tasks, builder):
    return UnifiedModelInfo(name, ModelCategory.Language, arch, params, params * 2, desc, tasks, builder)


def list_all_models() -> list:
    from .. import llm, vision
    L, V = llm, vision
    return [
        _v("lenet5", "LeNet", 61_706, "LeNet-5 for 28x28 digits", ("classification",), V.LeNet.new),
        _v("simple_cnn", "SimpleCNN", 421_642, "two-conv CNN", ("classification",), V.SimpleCNN.for_mnist),
        _v("mlp_mnist", "MLP", 235_146, "784-256-128-10 MLP", ("classification",), V.MLP.for_mnist),
        _v("resnet18", "ResNet", 11_689_512, "ResNet-18", ("classification",), V.resnet18),
        _v("resnet34", "ResNet", 21_797_672, "ResNet-34", ("classification",), V.resnet34),
        _v("vgg11", "VGG", 132_863_336, "VGG-11", ("classification",), V.vgg11),
        _v("vgg16", "VGG", 138_357_544, "VGG-16", ("classification",), V.vgg16),
        _v("vgg19", "VGG", 143_667_240, "VGG-19", ("classification",), V.vgg19),
        _v("vit_tiny", "ViT", 5_700_000, "ViT-Tiny/16", ("classification",), V.VisionTransformer.vit_tiny),
        _v("vit_base", "ViT", 86_000_000, "ViT-Base/16", ("classification",), V.VisionTransformer.vit_base),
        _l("gpt2", "GPT2", 124_000_000, "GPT-2 small", ("generation",), lambda: L.GPT2LMHead(L.GPT2Config.small())),
        _l("gpt2-medium", "GPT2", 355_000_000, "GPT-2 medium", ("generation",), lambda: L.GPT2LMHead(L.GPT2Config.medium())),
        _l("gpt2-large", "GPT2", 774_000_000, "GPT-2 large", ("generation",), lambda: L.GPT2LMHead(L.GPT2Config.large())),
        _l("gpt2-xl", "GPT2", 1_558_000_000, "GPT-2 XL", ("generation",), lambda: L.GPT2LMHead(L.GPT2Config.xl())),
        _l("gpt-1.3b", "GPT2", 1_316_000_000, "GPT-style 1.3B decoder", ("generation",), lambda: L.GPT2LMHead(L.GPT2Config.gpt_1_3b())),
        _l("llama2-7b", "LLaMA", 6_738_000_000, "LLaMA-2 7B", ("generation", "chat"), lambda: L.LLaMAForCausalLM(L.LLaMAConfig.llama2_7b())),
        _l("llama2-13b", "LLaMA", 13_016_000_000, "LLaMA-2 13B", ("generation", "chat"), lambda: L.LLaMAForCausalLM(L.LLaMAConfig.llama2_13b())),
        _l("llama3-8b", "LLaMA", 8_030_000_000, "LLaMA-3 8B", ("generation", "chat"), lambda: L.LLaMAForCausalLM(L.LLaMAConfig.llama3_8b())),
        _l("mistral-7b", "Mistral", 7_242_000_000, "Mistral 7B", ("generation",), lambda: L.MistralForCausalLM(L.MistralConfig.mistral_7b())),
        _l("phi-2", "Phi", 2_780_000_000, "Phi-2", ("generation", "code"), lambda: L.PhiForCausalLM(L.PhiConfig.phi2())),
        _l("bert-base", "BERT", 110_000_000, "BERT base uncased", ("embedding", "classification"), lambda: L.Bert(L.BertConfig.base())),
        _l("bert-large", "BERT", 340_000_000, "BERT large uncased", ("embedding", "classification"), lambda: L.Bert(L.BertConfig.large())),
    ]


def search_models(query: str) -> list:
    q = query.lower()
    return [m for m in list_all_models() if q in m.name.lower() or q in m.description.lower() or q in m.architecture.lower()]


def models_by_category(category: ModelCategory) -> list: return [m for m in list_all_models() if m.category is category]
def models_by_max_size_mb(max_mb: float) -> list: return [m for m in list_all_models() if m.size_mb() <= max_mb]
def models_by_max_params(max_params: int) -> list: return [m for m in list_all_models() if m.num_parameters <= max_params]
def recommended_models(task: str) -> list: return [m for m in list_all_models() if task.lower() in m.tasks]


def get_model_info(name: str):
    for m in list_all_models():
        if m.name == name:
            return m
    return None


# ------------------------------------------------------------------ cache + vision weight format
def cache_dir() -> str:
    d = os.environ.get("AXONML_HUB_CACHE", os.path.join(os.path.expanduser("~"), ".axonml", "hub"))
    os.makedirs(d, exist_ok=True)
    return d


def is_cached(name: str) -> bool: return os.path.exists(os.path.join(cache_dir(), name + ".weights"))


def save_hub_weights(tensors: dict, path) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<I", len(tensors)))
        for name, t in tensors.items():
            nb = name.encode()
            a = t.detach().cpu().float().contiguous().numpy()
            f.write(struct.pack("<I", len(nb)) + nb + struct.pack("<I", a.ndim) + struct.pack(f"<{a.ndim}Q", *a.shape))
            f.write(a.tobytes())


def load_hub_weights(path) -> dict:
    out = {}
    with open(path, "rb") as f:
        data = f.read()
    pos = 0
    (n,) = struct.unpack_from("<I", data, pos); pos += 4
    for _ in range(n):
        (ln,) = struct.unpack_from("<I", data, pos); pos += 4
        name = data[pos:pos + ln].decode(); pos += ln
        (nd,) = struct.unpack_from("<I", data, pos); pos += 4
        dims = struct.unpack_from(f"<{nd}Q", data, pos); pos += 8 * nd
        cnt = int(np.prod(dims)) if nd else 1
        out[name] = torch.from_numpy(np.frombuffer(data, dtype="<f4", count=cnt, offset=pos).copy()).view(dims)
        pos += 4 * cnt
    return out


def load_pretrained(name: str, **kw):
    """Builds the model and loads cached weights when present (no network is used)."""
    info = get_model_info(name)
    if info is None:
        raise KeyError(name)
    model = info.build(**kw)
    p = os.path.join(cache_dir(), name + ".weights")
    if os.path.exists(p):
        sd = load_hub_weights(p)
        own = dict(model.named_parameters())
        with torch.no_grad():
            for k, v in sd.items():
                if k in own and own[k].shape == v.shape:
                    own[k].copy_(v)
    return model
