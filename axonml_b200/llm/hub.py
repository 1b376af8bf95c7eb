"""Registry of pretrained language models and their weight cache.

Parity: crates/axonml-llm/src/hub.rs (``PretrainedLLM{name, url, checksum, size_bytes, vocab_size,
hidden_size, num_layers, num_heads, max_seq_len, num_parameters, architecture, dataset}``,
``llm_registry`` with the BERT, GPT-2, DistilBERT, RoBERTa, ALBERT, LLaMA, Mistral, Phi and Qwen
entries, ``cache_dir`` = ``<cache>/axonml/hub/llm``, ``is_cached`` / ``cached_path``
(``<name>.safetensors``), ``download_weights(name, force)``, ``list_models``, ``model_info``,
``models_by_architecture`` (case-insensitive), ``models_by_max_params`` (ascending)).  The figures
are the published architecture sizes of each model."""
from __future__ import annotations

import dataclasses
import os

from ..hub.download import HubError, ModelNotFound, fetch, format_params, hub_cache_root, repo_url  # noqa: F401


@dataclasses.dataclass(frozen=True)
class PretrainedLLM:
    name: str
    repo: str                     # <org>/<repository> on the hub
    size_bytes: int
    vocab_size: int
    hidden_size: int
    num_layers: int
    num_heads: int
    max_seq_len: int
    num_parameters: int
    architecture: str
    dataset: str
    checksum: str | None = None
    filename: str = "model.safetensors"

    @property
    def url(self) -> str:
        return repo_url(self.repo, self.filename)

    def params_str(self) -> str:
        return format_params(self.num_parameters)


def _e(name, repo, mb, vocab, hidden, layers, heads, seq, params, arch, dataset):
    return PretrainedLLM(name, repo, int(mb * 1_000_000), vocab, hidden, layers, heads, seq, int(params), arch, dataset)


_OWN = "axonml-ml/"
_ENTRIES = [
    # name, repository, file MB, vocabulary, hidden, layers, heads, context, parameters, architecture, corpus
    _e("bert-tiny", _OWN + "bert-tiny", 17, 30522, 128, 2, 2, 512, 4.4e6, "BERT", "BookCorpus + Wikipedia"),
    _e("bert-mini", _OWN + "bert-mini", 45, 30522, 256, 4, 4, 512, 11.3e6, "BERT", "BookCorpus + Wikipedia"),
    _e("bert-base-uncased", _OWN + "bert-base-uncased", 440, 30522, 768, 12, 12, 512, 110e6, "BERT", "BookCorpus + Wikipedia"),
    _e("bert-base-cased", _OWN + "bert-base-cased", 436, 28996, 768, 12, 12, 512, 108e6, "BERT", "BookCorpus + Wikipedia"),
    _e("bert-large-uncased", _OWN + "bert-large-uncased", 1340, 30522, 1024, 24, 16, 512, 340e6, "BERT", "BookCorpus + Wikipedia"),
    _e("gpt2", _OWN + "gpt2", 548, 50257, 768, 12, 12, 1024, 124e6, "GPT2", "WebText"),
    _e("gpt2-medium", _OWN + "gpt2-medium", 1520, 50257, 1024, 24, 16, 1024, 355e6, "GPT2", "WebText"),
    _e("gpt2-large", _OWN + "gpt2-large", 3250, 50257, 1280, 36, 20, 1024, 774e6, "GPT2", "WebText"),
    _e("gpt2-xl", _OWN + "gpt2-xl", 6430, 50257, 1600, 48, 25, 1024, 1558e6, "GPT2", "WebText"),
    _e("distilbert-base-uncased", _OWN + "distilbert-base-uncased", 268, 30522, 768, 6, 12, 512, 66e6, "DistilBERT",
       "BookCorpus + Wikipedia (distilled from BERT base)"),
    _e("roberta-base", _OWN + "roberta-base", 500, 50265, 768, 12, 12, 514, 125e6, "RoBERTa", "BookCorpus, CC-News, OpenWebText, Stories"),
    _e("roberta-large", _OWN + "roberta-large", 1420, 50265, 1024, 24, 16, 514, 355e6, "RoBERTa", "BookCorpus, CC-News, OpenWebText, Stories"),
    _e("albert-base-v2", _OWN + "albert-base-v2", 47, 30000, 768, 12, 12, 512, 11.7e6, "ALBERT", "BookCorpus + Wikipedia"),
    _e("albert-large-v2", _OWN + "albert-large-v2", 71, 30000, 1024, 24, 16, 512, 17.7e6, "ALBERT", "BookCorpus + Wikipedia"),
    _e("llama-2-7b", "meta-llama/Llama-2-7b-hf", 13_500, 32000, 4096, 32, 32, 4096, 6.74e9, "LLaMA", "2T tokens of public text"),
    _e("llama-2-13b", "meta-llama/Llama-2-13b-hf", 26_000, 32000, 5120, 40, 40, 4096, 13.0e9, "LLaMA", "2T tokens of public text"),
    _e("tinyllama-1.1b", "TinyLlama/TinyLlama-1.1B-Chat-v1.0", 2200, 32000, 2048, 22, 32, 2048, 1.1e9, "LLaMA", "SlimPajama + StarCoder data"),
    _e("mistral-7b", "mistralai/Mistral-7B-v0.1", 14_500, 32000, 4096, 32, 32, 32768, 7.24e9, "Mistral", "undisclosed web text"),
    _e("mistral-7b-instruct", "mistralai/Mistral-7B-Instruct-v0.2", 14_500, 32000, 4096, 32, 32, 32768, 7.24e9, "Mistral",
       "Mistral 7B + instruction tuning"),
    _e("phi-2", "microsoft/phi-2", 5560, 51200, 2560, 32, 32, 2048, 2.78e9, "Phi", "synthetic textbooks + filtered web"),
    _e("phi-1.5", "microsoft/phi-1_5", 2840, 51200, 2048, 24, 32, 2048, 1.42e9, "Phi", "synthetic textbooks"),
    _e("qwen-1.8b", "Qwen/Qwen-1_8B", 3670, 151936, 2048, 24, 16, 8192, 1.84e9, "Qwen", "2.2T multilingual tokens"),
    _e("qwen-7b", "Qwen/Qwen-7B", 15_400, 151936, 4096, 32, 32, 8192, 7.72e9, "Qwen", "2.4T multilingual tokens"),
]


def llm_registry() -> dict:
    return {m.name: m for m in _ENTRIES}


def cache_dir() -> str:
    return os.path.join(hub_cache_root(), "llm")


def cached_path(model_name: str) -> str:
    return os.path.join(cache_dir(), model_name + ".safetensors")


def is_cached(model_name: str) -> bool:
    return os.path.exists(cached_path(model_name))


def download_weights(model_name: str, force: bool = False, quiet: bool = False) -> str:
    """Path of the model's weights, downloading them first unless already cached."""
    info = llm_registry().get(model_name)
    if info is None:
        raise ModelNotFound(model_name)
    path = cached_path(model_name)
    if os.path.exists(path) and not force:
        return path
    if not quiet:
        print(f"Downloading {model_name} ({info.size_bytes / 1e6:.1f} MB, {info.params_str()} parameters)...")
    fetch(info.url, path, info.checksum)
    if not quiet:
        print(f"Downloaded to {path}")
    return path


def list_models() -> list:
    return list(_ENTRIES)


def model_info(name: str):
    return llm_registry().get(name)


def models_by_architecture(arch: str) -> list:
    return [m for m in _ENTRIES if m.architecture.lower() == arch.lower()]


def models_by_max_params(max_params: int) -> list:
    return sorted((m for m in _ENTRIES if m.num_parameters <= max_params), key=lambda m: m.num_parameters)
