"""LLaMA family (crates/axonml-llm/src/llama.rs): RMSNorm, rotary embedding in the half-split
convention (:208-322), grouped-query attention (:330-496), SwiGLU MLP (:542-567), decoder layer,
``LLaMA`` and ``LLaMAForCausalLM``.  Weight names are the HuggingFace ones
(``embed_tokens.weight``, ``layers.{i}.self_attn.{q,k,v,o}_proj.weight``,
``layers.{i}.mlp.{gate,up,down}_proj.weight``, ``layers.{i}.input_layernorm.weight``,
``layers.{i}.post_attention_layernorm.weight``, ``norm.weight``, ``lm_head.weight``); all Linears
are bias-free.

B200 execution: q/k/v are computed by ONE GEMM on the row-concatenated weights (the three
parameters stay separate for checkpoints; the concatenation is a cached view rebuilt when a
weight changes), gate/up likewise, SwiGLU and RoPE are hand-written kernels, residual adds are
fused into RMSNorm, attention is the GQA-aware flash kernel on the token-major tensors."""
from __future__ import annotations

import torch

from .. import nn
from ..autograd.checkpoint import checkpoint
from ..ops import elementwise as E
from ..ops import loss as L
from ..ops import misc as Mi
from ..ops.attention import sdpa, sdpa_packed
from ..ops.linear import linear
from .attention import LayerKVCache
from .config import LLaMAConfig
from ._api import ModelApi
from .hf_loader import LoadStateDict


class RotaryEmbedding(nn.Module):
    def __init__(self, head_dim: int, max_position_embeddings: int, theta: float = 10000.0):
        super().__init__()
        self.head_dim, self.max_pos, self.theta = head_dim, max_position_embeddings, theta
        cos, sin = Mi.rope_tables(max_position_embeddings, head_dim, theta)
        self.register_buffer("cos_cached", cos, persistent=False)
        self.register_buffer("sin_cached", sin, persistent=False)

    def apply(self, x: torch.Tensor, seq_len: int, pos0: int = 0) -> torch.Tensor:  # type: ignore[override]
        """``x [B, S, H, D]`` -> rotated."""
        if self.cos_cached.device != x.device:
            self.cos_cached = self.cos_cached.to(x.device)
            self.sin_cached = self.sin_cached.to(x.device)
        return Mi.rope(x, self.cos_cached, self.sin_cached, seq_len=seq_len, pos0=pos0)


def _cat_rows(*ws):
    return torch.cat(ws, dim=0)


class LLaMAAttention(nn.Module):
    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        self.nh, self.nkv, self.hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim()
        H = cfg.hidden_size
        self.q_proj = nn.Linear(H, self.nh * self.hd, bias=False, device=device, dtype=dtype)
        self.k_proj = nn.Linear(H, self.nkv * self.hd, bias=False, device=device, dtype=dtype)
        self.v_proj = nn.Linear(H, self.nkv * self.hd, bias=False, device=device, dtype=dtype)
        self.o_proj = nn.Linear(self.nh * self.hd, H, bias=False, device=device, dtype=dtype)
        self.rotary = RotaryEmbedding(self.hd, cfg.max_position_embeddings, cfg.rope_theta)
        self.sliding_window = getattr(cfg, "sliding_window", None)

    def forward(self, x, kv_cache=None, pos0: int = 0):
        B, S, _ = x.shape
        w = _cat_rows(self.q_proj.weight, self.k_proj.weight, self.v_proj.weight)
        qkv = linear(x, w)
        cp = getattr(self, "cp_group", None)
        if cp is not None and kv_cache is None and self.sliding_window is None:
            # context parallel: x holds this rank's slice of the sequence; positions continue from
            # the slices before it and attention runs over the whole sequence
            from ..parallel import context_parallel as CP
            nq, nk = self.nh * self.hd, self.nkv * self.hd
            p0 = pos0 + cp.rank() * S
            q = self.rotary.apply(qkv[..., :nq].reshape(B, S, self.nh, self.hd), S, p0)
            k = self.rotary.apply(qkv[..., nq:nq + nk].reshape(B, S, self.nkv, self.hd), S, p0)
            v = qkv[..., nq + nk:].reshape(B, S, self.nkv, self.hd)
            attend = CP.attention_fn(getattr(self, "cp_form", "ulysses"))
            o = attend(q.contiguous(), k.contiguous(), v.contiguous(), cp, causal=True)
            return self.o_proj(o.reshape(B, S, self.nh * self.hd))
        if kv_cache is None and self.sliding_window is None:
            packed = qkv.view(B, S, self.nh + 2 * self.nkv, self.hd)
            packed = Mi.rope(packed, self.rotary.cos_cached.to(x.device), self.rotary.sin_cached.to(x.device),
                             seq_len=S, pos0=pos0, rot_heads=self.nh + self.nkv)
            o = sdpa_packed(packed, self.nh, self.nkv, causal=True)
            return self.o_proj(o.reshape(B, S, self.nh * self.hd))
        nq, nk = self.nh * self.hd, self.nkv * self.hd
        q = qkv[..., :nq].reshape(B, S, self.nh, self.hd)
        k = qkv[..., nq:nq + nk].reshape(B, S, self.nkv, self.hd)
        v = qkv[..., nq + nk:].reshape(B, S, self.nkv, self.hd)
        q = self.rotary.apply(q, S, pos0)
        k = self.rotary.apply(k, S, pos0)
        if kv_cache is not None:
            k, v = kv_cache.update(k, v)
        mask = None
        if self.sliding_window is not None and k.shape[1] > self.sliding_window:
            Sk = k.shape[1]
            i = torch.arange(Sk - S, Sk, device=x.device)[:, None]
            j = torch.arange(Sk, device=x.device)[None, :]
            mask = (j <= i) & (j > i - self.sliding_window)
            o = sdpa(q, k, v, mask=mask)
        else:
            o = sdpa(q, k, v, causal=True)
        return self.o_proj(o.reshape(B, S, self.nh * self.hd))


    def forward_with_cache(self, x, kv_cache, pos0: int | None = None):
        """Attention over ``x`` appended to ``kv_cache``; positions continue from the cache."""
        return self.forward(x, kv_cache, kv_cache.seq_len if pos0 is None and kv_cache is not None else (pos0 or 0))


class LLaMAMLP(nn.Module):
    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.gate_proj = nn.Linear(H, I, bias=False, device=device, dtype=dtype)
        self.up_proj = nn.Linear(H, I, bias=False, device=device, dtype=dtype)
        self.down_proj = nn.Linear(I, H, bias=False, device=device, dtype=dtype)

    def forward(self, x):
        gu = linear(x, _cat_rows(self.gate_proj.weight, self.up_proj.weight))
        return self.down_proj(E.swiglu(gu))


class LLaMADecoderLayer(nn.Module):
    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        self.input_layernorm = nn.RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device, dtype=dtype)
        self.self_attn = LLaMAAttention(cfg, device, dtype)
        self.post_attention_layernorm = nn.RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device, dtype=dtype)
        self.mlp = LLaMAMLP(cfg, device, dtype)

    def forward(self, delta, residual=None, kv_cache=None, pos0: int = 0):
        if residual is None:
            a, residual = self.input_layernorm(delta), delta
        else:
            a, residual = self.input_layernorm(delta, residual=residual)
        attn = self.self_attn(a, kv_cache, pos0)
        m, residual = self.post_attention_layernorm(attn, residual=residual)
        return self.mlp(m), residual

    def forward_with_cache(self, x, kv_cache, pos0: int | None = None):
        """The whole layer on a hidden state ``x`` (residual connections included), appending to ``kv_cache``."""
        p = kv_cache.seq_len if pos0 is None and kv_cache is not None else (pos0 or 0)
        delta, residual = self.forward(x, None, kv_cache, p)
        return delta + residual


class LLaMA(nn.Module, ModelApi):
    ARCH = "llama"

    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, device=device, dtype=dtype)
        self.layers = nn.ModuleList([LLaMADecoderLayer(cfg, device, dtype) for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device, dtype=dtype)
        self.gradient_checkpointing = False
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, 0.02)

    @classmethod
    def new(cls, cfg): return cls(cfg)

    def forward(self, ids, kv_caches=None, pos0: int = 0):
        delta, residual = self.embed_tokens(ids), None
        for i, layer in enumerate(self.layers):
            cache = kv_caches[i] if kv_caches is not None else None
            if self.gradient_checkpointing and self.training and cache is None:
                if residual is None:
                    delta, residual = checkpoint(lambda d, l=layer: l(d), delta)
                else:
                    delta, residual = checkpoint(layer, delta, residual)
            else:
                delta, residual = layer(delta, residual, cache, pos0)
        h, _ = self.norm(delta, residual=residual)
        return h

    def create_kv_cache(self, batch: int, max_seq_len: int | None = None):
        p = next(self.parameters())
        return LayerKVCache(self.cfg.num_hidden_layers, batch, max_seq_len or self.cfg.max_position_embeddings,
                            self.cfg.num_key_value_heads, self.cfg.head_dim(), device=p.device, dtype=p.dtype)

    @classmethod
    def _config_from_json(cls, j):
        from .hf_loader import parse_llama_config_from_json
        return parse_llama_config_from_json(j)


class LLaMAForCausalLM(nn.Module, LoadStateDict, ModelApi):
    ARCH = "llama"

    def __init__(self, cfg: LLaMAConfig, tie_word_embeddings: bool = False, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.model = LLaMA(cfg, device, dtype)
        self.tied = tie_word_embeddings
        if not tie_word_embeddings:
            self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, device=device, dtype=dtype)
            with torch.no_grad():
                self.lm_head.weight.normal_(0.0, 0.02)

    @classmethod
    def new(cls, cfg): return cls(cfg)

    def gradient_checkpointing_enable(self, flag: bool = True):
        self.model.gradient_checkpointing = flag
        return self

    def create_kv_cache(self, batch: int, max_seq_len: int | None = None):
        p = next(self.parameters())
        return LayerKVCache(self.cfg.num_hidden_layers, batch, max_seq_len or self.cfg.max_position_embeddings,
                            self.cfg.num_key_value_heads, self.cfg.head_dim(), device=p.device, dtype=p.dtype)

    def head_weight(self):
        return self.model.embed_tokens.weight if self.tied else self.lm_head.weight

    def forward(self, ids, kv_caches=None, pos0: int = 0):
        return linear(self.model(ids, kv_caches, pos0), self.head_weight())

    @classmethod
    def _config_from_json(cls, j):
        from .hf_loader import parse_llama_config_from_json
        return parse_llama_config_from_json(j)

    def enable_context_parallel(self, process_group, form: str = "ulysses"):
        """Shards the sequence over ``process_group``: ``forward_with_loss`` then takes the whole
        sequence on every rank, runs this rank's slice (``form``: "ulysses" all-to-all,
        "allgather" of K/V or "ring") and returns a loss whose mean over the ranks is the loss of the whole
        sequence, so a data-parallel wrapper's gradient average over the same ranks is exact."""
        from ..parallel.context_parallel import attention_fn
        attention_fn(form)                                   # validates the name
        self.cp_group = process_group
        for layer in self.model.layers:
            layer.self_attn.cp_group, layer.self_attn.cp_form = process_group, form
        return self

    def forward_with_loss(self, ids, labels=None):
        labels = ids if labels is None else labels
        cp = getattr(self, "cp_group", None)
        if cp is not None and cp.world_size() > 1:
            from ..parallel.context_parallel import shard_sequence
            tgt = torch.full_like(labels, -100)
            tgt[:, :-1] = labels[:, 1:]
            total = (tgt != -100).sum().clamp_min(1)
            logits = self.forward(shard_sequence(ids, cp))
            tl = shard_sequence(tgt, cp).reshape(-1)
            B, S, V = logits.shape
            local = (tl != -100).sum()
            loss = L.cross_entropy(logits.view(B * S, V), tl) * (local * cp.world_size() / total)
            return loss, logits
        logits = self.forward(ids)
        B, S, V = logits.shape
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
        return L.cross_entropy(logits.view(B * S, V), tgt.view(-1)), logits

    @torch.no_grad()
    def generate(self, ids, max_new_tokens: int = 20, temperature: float = 1.0, top_k=None, eos_token_id=None):
        from .generation import GenerationConfig, TextGenerator
        cfg = GenerationConfig(max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k,
                               do_sample=(temperature != 1.0 or top_k is not None),
                               eos_token_ids=[eos_token_id] if eos_token_id is not None else [])
        return TextGenerator(cfg).generate(self, ids)

    def load_state_dict_hf(self, sd: dict, strict: bool = False):
        """Accepts HuggingFace keys with or without the ``model.`` prefix; ties ``lm_head`` to the
        embeddings when it is absent (llama.rs:782-822)."""
        own = dict(self.named_parameters())
        missing = []
        for name, p in own.items():
            cands = [name, name.removeprefix("model."), "model." + name]
            src = next((sd[c] for c in cands if c in sd), None)
            if src is None and name == "lm_head.weight":
                src = sd.get("model.embed_tokens.weight", sd.get("embed_tokens.weight"))
            if src is None:
                missing.append(name)
                continue
            with torch.no_grad():
                p.copy_(torch.as_tensor(src).to(p.dtype))
        if strict and missing:
            raise KeyError(f"missing keys: {missing}")
        return missing
