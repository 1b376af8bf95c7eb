"""Mistral (sliding-window attention, grouped-query heads; crates/axonml-llm/src/mistral.rs) and Phi
(partial rotary embedding, parallel attention + MLP block, LayerNorm; phi.rs)."""
from __future__ import annotations

import torch

from .. import nn
from ..ops import misc as Mi
from ..ops.attention import sdpa
from ..ops.linear import linear
from .attention import LayerKVCache
from .config import MistralConfig, PhiConfig
from ._api import ModelApi
from .hf_loader import LoadStateDict
from .llama import LLaMAForCausalLM


class MistralForCausalLM(LLaMAForCausalLM):
    """Same decoder as LLaMA; ``cfg.sliding_window`` limits every query to the last W keys."""

    ARCH = "mistral"

    def __init__(self, cfg: MistralConfig, **kw):
        super().__init__(cfg, **kw)

    @classmethod
    def new(cls, cfg): return cls(cfg)

    @classmethod
    def _config_from_json(cls, j):
        from .hf_loader import parse_mistral_config
        return parse_mistral_config(j)


Mistral = MistralForCausalLM
# the blocks are LLaMA's (grouped-query attention with the window taken from the config, SwiGLU MLP);
# the reference names them per family (mistral.rs: MistralAttention, MistralMLP, MistralDecoderLayer)
from .llama import LLaMAAttention as MistralAttention  # noqa: E402
from .llama import LLaMADecoderLayer as MistralDecoderLayer  # noqa: E402
from .llama import LLaMAMLP as MistralMLP  # noqa: E402


class PhiAttention(nn.Module):
    def __init__(self, cfg: PhiConfig):
        super().__init__()
        self.nh, self.nkv, self.hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim()
        H = cfg.hidden_size
        self.q_proj, self.k_proj = nn.Linear(H, self.nh * self.hd), nn.Linear(H, self.nkv * self.hd)
        self.v_proj, self.dense = nn.Linear(H, self.nkv * self.hd), nn.Linear(self.nh * self.hd, H)
        self.rot = int(self.hd * cfg.partial_rotary_factor) // 2 * 2
        cos, sin = Mi.rope_tables(cfg.max_position_embeddings, max(self.rot, 2), cfg.rope_theta)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def _rope(self, x, S, pos0):
        if self.rot == 0:
            return x
        a = Mi.rope(x[..., :self.rot].contiguous(), self.cos.to(x.device), self.sin.to(x.device), seq_len=S, pos0=pos0)
        return torch.cat([a, x[..., self.rot:]], dim=-1)

    def forward(self, x, kv_cache=None, pos0=0):
        B, S, _ = x.shape
        q = self._rope(self.q_proj(x).view(B, S, self.nh, self.hd), S, pos0)
        k = self._rope(self.k_proj(x).view(B, S, self.nkv, self.hd), S, pos0)
        v = self.v_proj(x).view(B, S, self.nkv, self.hd)
        if kv_cache is not None:
            k, v = kv_cache.update(k, v)
        return self.dense(sdpa(q, k, v, causal=True).reshape(B, S, self.nh * self.hd))

    def forward_with_cache(self, x, kv_cache, pos0: int | None = None):
        return self.forward(x, kv_cache, kv_cache.seq_len if pos0 is None and kv_cache is not None else (pos0 or 0))


class PhiMLP(nn.Module):
    """fc1 -> GELU -> fc2 (phi.rs ``PhiMLP``); the activation runs in the first GEMM's epilogue."""

    def __init__(self, cfg: PhiConfig):
        super().__init__()
        self.fc1 = nn.Linear(cfg.hidden_size, cfg.intermediate_size, activation="gelu")
        self.fc2 = nn.Linear(cfg.intermediate_size, cfg.hidden_size)

    def forward(self, x):
        return self.fc2(self.fc1(x))


class PhiDecoderLayer(nn.Module):
    def __init__(self, cfg: PhiConfig):
        super().__init__()
        self.parallel = cfg.parallel_attn
        self.input_layernorm = nn.LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.post_layernorm = None if self.parallel else nn.LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.self_attn = PhiAttention(cfg)
        self.mlp = PhiMLP(cfg)

    def forward(self, x, kv_cache=None, pos0=0):
        h = self.input_layernorm(x)
        a = self.self_attn(h, kv_cache, pos0)
        if self.parallel:
            return x + a + self.mlp(h)
        x = x + a
        return x + self.mlp(self.post_layernorm(x))

    def forward_with_cache(self, x, kv_cache, pos0: int | None = None):
        return self.forward(x, kv_cache, kv_cache.seq_len if pos0 is None and kv_cache is not None else (pos0 or 0))


class PhiForCausalLM(nn.Module, LoadStateDict, ModelApi):
    ARCH = "phi"

    def __init__(self, cfg: PhiConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([PhiDecoderLayer(cfg) for _ in range(cfg.num_hidden_layers)])
        self.final_layernorm = nn.LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size)

    @classmethod
    def new(cls, cfg): return cls(cfg)

    def create_kv_cache(self, batch, max_seq_len=None):
        p = next(self.parameters())
        return LayerKVCache(self.cfg.num_hidden_layers, batch, max_seq_len or self.cfg.max_position_embeddings,
                            self.cfg.num_key_value_heads, self.cfg.head_dim(), device=p.device, dtype=p.dtype)

    def forward(self, ids, kv_caches=None, pos0=0):
        h = self.embed_tokens(ids)
        for i, l in enumerate(self.layers):
            h = l(h, kv_caches[i] if kv_caches is not None else None, pos0)
        return self.lm_head(self.final_layernorm(h))

    @classmethod
    def with_parallel_attn(cls, cfg: PhiConfig, parallel: bool = True):
        """Model whose blocks run attention and MLP side by side on the same normalised input
        (``parallel=True``, Phi-1 / Phi-2) or one after the other."""
        import dataclasses
        return cls(dataclasses.replace(cfg, parallel_attn=parallel))

    @classmethod
    def _config_from_json(cls, j):
        d = PhiConfig()
        head = int(j.get("num_attention_heads", d.num_attention_heads))
        return PhiConfig(vocab_size=int(j.get("vocab_size", d.vocab_size)), hidden_size=int(j.get("hidden_size", d.hidden_size)),
                         intermediate_size=int(j.get("intermediate_size", d.intermediate_size)),
                         num_hidden_layers=int(j.get("num_hidden_layers", d.num_hidden_layers)), num_attention_heads=head,
                         num_key_value_heads=int(j.get("num_key_value_heads") or head),
                         max_position_embeddings=int(j.get("max_position_embeddings", d.max_position_embeddings)),
                         layer_norm_eps=float(j.get("layer_norm_eps", d.layer_norm_eps)), rope_theta=float(j.get("rope_theta", d.rope_theta)),
                         partial_rotary_factor=float(j.get("partial_rotary_factor", d.partial_rotary_factor)))


Phi = PhiForCausalLM
