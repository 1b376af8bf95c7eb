"""Methods every language model of the package answers under the reference's names.

Parity: the ``forward_ids`` / ``forward_with_cache`` / ``config`` / ``from_pretrained`` /
``generate_greedy`` methods of crates/axonml-llm/src/{llama,mistral,phi,gpt2,bert}.rs.  The classes
mix this in; each keeps its own ``forward``."""
from __future__ import annotations

import os

import torch


class ModelApi:
    ARCH = ""                                   # family name the weight mappers know: "llama", "mistral", "phi", "gpt2", "bert"

    def config(self):
        """The configuration the model was built from."""
        return self.cfg

    def forward_ids(self, ids, *args, **kw):
        """``forward`` for token ids of any integer (or, as in the reference, float) type."""
        ids = torch.as_tensor(ids)
        if ids.dim() == 1:
            ids = ids.unsqueeze(0)
        return self.forward(ids.long(), *args, **kw)

    def forward_with_cache(self, ids, kv_caches=None, pos0: int | None = None):
        """One decoding step over ``ids`` that appends to ``kv_caches`` (``create_kv_cache``);
        positions continue from what the cache already holds unless ``pos0`` is given."""
        if kv_caches is not None and pos0 is None:
            pos0 = kv_caches.seq_len() if hasattr(kv_caches, "seq_len") else 0
        return self.forward(ids, kv_caches, pos0 or 0)

    @torch.no_grad()
    def generate_greedy(self, ids, max_new_tokens: int = 20, eos_token_id=None):
        from .generation import GenerationConfig, TextGenerator
        cfg = GenerationConfig.greedy(max_new_tokens)
        if eos_token_id is not None:
            cfg.with_eos_token(eos_token_id)
        return TextGenerator(cfg).generate(self, ids)

    @classmethod
    def _config_from_json(cls, j: dict):
        raise NotImplementedError

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, strict: bool = False, device=None, dtype=None):
        """Model with the configuration and weights of a checkpoint directory or hub model id
        (``config.json`` + safetensors)."""
        from .hf_loader import HFLoader, load_with_mapping
        loader = HFLoader.from_local(model_id_or_path) if os.path.isdir(model_id_or_path) else HFLoader.new(model_id_or_path)
        cfg = cls._config_from_json(loader.load_config())
        model = cls(cfg)
        weights = {k: v for k, v in loader.load_tensors().items() if "rotary_emb.inv_freq" not in k}
        load_with_mapping(model, weights, cls.ARCH, strict=strict)
        if device is not None or dtype is not None:
            model = model.to(device=device, dtype=dtype)
        return model.eval()
