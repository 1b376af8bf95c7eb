"""GPT-2 family (crates/axonml-llm/src/gpt2.rs:77-266, transformer.rs:229-430,
embedding.rs:335-365).  Pre-LN decoder: ``ln1 -> CausalSelfAttention -> +res -> ln2 ->
FeedForward(4d) -> +res``.  State-dict keys follow the reference's member names:
``wte.wte.weight``, ``wte.wpe.weight``, ``blocks.{i}.attention.c_attn.*``, ``.c_proj.*``,
``.ln1.*``, ``.ln2.*``, ``.ffn.fc1.*``, ``.ffn.fc2.*``, ``ln_f.*``; the LM head is tied to ``wte``.

B200 execution: every projection is the tcgen05 GEMM with its bias (and GELU) in the epilogue, the
residual adds are fused into the LayerNorm kernel (each block passes ``(delta, residual)`` to the
next), attention is the flash kernel on the token-major fused QKV tensor, the loss is the fused
cross-entropy over a vocabulary padded to a multiple of 128 for the GEMM."""
from __future__ import annotations

import torch

from .. import nn
from ..autograd.checkpoint import checkpoint
from ..ops import loss as L
from ..ops import misc as Mi
from ..ops.attention import sdpa, sdpa_packed
from ..ops.linear import linear
from .config import GPT2Config
from ._api import ModelApi
from .hf_loader import LoadStateDict


class GPT2Embedding(nn.Module):
    """Token + learned position embeddings (+ dropout)."""

    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.vocab_padded = cfg.padded_vocab()
        self.wte = nn.Embedding(self.vocab_padded, cfg.n_embd, device=device, dtype=dtype)
        self.wpe = nn.Embedding(cfg.n_ctx, cfg.n_embd, device=device, dtype=dtype)
        self.drop = nn.Dropout(cfg.dropout)
        with torch.no_grad():
            self.wte.weight.normal_(0.0, 0.02)
            self.wte.weight[cfg.vocab_size:].zero_()
            self.wpe.weight.normal_(0.0, 0.02)

    def forward(self, ids: torch.Tensor, pos0: int = 0) -> torch.Tensor:
        B, S = ids.shape
        x = Mi.embedding(ids, self.wte.weight, pos_weight=self.wpe.weight, seq_len=S, pos0=pos0)
        return self.drop(x)

    def forward_ids(self, input_ids, pos0: int = 0):
        """Token + position embeddings of integer (or float-typed) ids."""
        ids = torch.as_tensor(input_ids)
        return self.forward((ids.unsqueeze(0) if ids.dim() == 1 else ids).long(), pos0)


class CausalSelfAttention(nn.Module):
    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        self.n_head, self.head_dim = cfg.n_head, cfg.head_dim()
        self.c_attn = nn.Linear(cfg.n_embd, 3 * cfg.n_embd, device=device, dtype=dtype)
        self.c_proj = nn.Linear(cfg.n_embd, cfg.n_embd, device=device, dtype=dtype)
        self.attn_dropout = cfg.attn_dropout
        self.resid_drop = nn.Dropout(cfg.resid_dropout)

    def forward(self, x, kv_cache=None):
        B, S, E = x.shape
        drop = self.attn_dropout if self.training else 0.0
        cp = getattr(self, "cp_group", None)
        if cp is not None and kv_cache is None:
            # context parallel: x is this rank's slice of the sequence, attention sees all of it
            from ..parallel import context_parallel as CP
            if drop > 0.0:
                raise ValueError("context-parallel attention does not support attention dropout")
            qkv = self.c_attn(x).view(B, S, 3, self.n_head, self.head_dim)
            attend = CP.attention_fn(getattr(self, "cp_form", "ulysses"))
            o = attend(qkv[:, :, 0].contiguous(), qkv[:, :, 1].contiguous(), qkv[:, :, 2].contiguous(), cp, causal=True)
        elif kv_cache is None:
            qkv = self.c_attn(x).view(B, S, 3 * self.n_head, self.head_dim)
            o = sdpa_packed(qkv, self.n_head, self.n_head, causal=True, dropout_p=drop)
        else:
            qkv = self.c_attn(x).view(B, S, 3, self.n_head, self.head_dim)
            q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
            k, v = kv_cache.update(k, v)
            o = sdpa(q, k, v, causal=True, dropout_p=drop)
        return self.resid_drop(self.c_proj(o.reshape(B, S, E)))

    def create_causal_mask(self, seq_len: int, device=None) -> torch.Tensor:
        """Additive mask [seq, seq]: 0 where query i may see key j (j <= i), -inf elsewhere."""
        m = torch.full((seq_len, seq_len), float("-inf"), device=device)
        return torch.triu(m, diagonal=1)

    def forward_causal(self, x):
        """Causal self-attention over a whole sequence (no cache)."""
        return self.forward(x, None)

    def forward_with_cache(self, x, kv_cache):
        """Attention of the new positions ``x`` over everything in ``kv_cache`` plus themselves."""
        return self.forward(x, kv_cache)


class FeedForward(nn.Module):
    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        act = {"gelu": "gelu", "relu": "relu", "silu": "silu", "swish": "silu", "tanh": "tanh"}[cfg.activation]
        self.fc1 = nn.Linear(cfg.n_embd, cfg.intermediate_size(), activation=act, device=device, dtype=dtype)
        self.fc2 = nn.Linear(cfg.intermediate_size(), cfg.n_embd, device=device, dtype=dtype)
        self.drop = nn.Dropout(cfg.resid_dropout)

    def forward(self, x):
        return self.drop(self.fc2(self.fc1(x)))


class TransformerBlock(nn.Module):
    """Takes and returns ``(delta, residual)``: the running residual stream is ``residual +
    delta``; the add is done inside the next LayerNorm kernel."""

    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        self.ln1 = nn.LayerNorm(cfg.n_embd, cfg.layer_norm_eps, device=device, dtype=dtype)
        self.attention = CausalSelfAttention(cfg, device, dtype)
        self.ln2 = nn.LayerNorm(cfg.n_embd, cfg.layer_norm_eps, device=device, dtype=dtype)
        self.ffn = FeedForward(cfg, device, dtype)

    def forward(self, delta, residual=None, kv_cache=None):
        if residual is None:
            a, residual = self.ln1(delta), delta
        else:
            a, residual = self.ln1(delta, residual=residual)
        attn = self.attention(a, kv_cache)
        m, residual = self.ln2(attn, residual=residual)
        return self.ffn(m), residual


class _Presets:
    """``Model.small()`` ... ``Model.tiny()``: the model built from the configuration preset of that name."""

    @classmethod
    def small(cls): return cls(GPT2Config.small())
    @classmethod
    def medium(cls): return cls(GPT2Config.medium())
    @classmethod
    def large(cls): return cls(GPT2Config.large())
    @classmethod
    def xl(cls): return cls(GPT2Config.xl())
    @classmethod
    def tiny(cls): return cls(GPT2Config.tiny())


class GPT2(nn.Module, ModelApi, _Presets):
    ARCH = "gpt2"

    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.wte = GPT2Embedding(cfg, device, dtype)
        self.blocks = nn.ModuleList([TransformerBlock(cfg, device, dtype) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.n_embd, cfg.layer_norm_eps, device=device, dtype=dtype)
        self.gradient_checkpointing = False
        self._init_weights()

    @classmethod
    def new(cls, cfg: GPT2Config): return cls(cfg)

    def _init_weights(self):
        std = 0.02
        with torch.no_grad():
            for blk in self.blocks:
                for lin in (blk.attention.c_attn, blk.attention.c_proj, blk.ffn.fc1, blk.ffn.fc2):
                    lin.weight.normal_(0.0, std)
                for lin in (blk.attention.c_proj, blk.ffn.fc2):
                    lin.weight.mul_(1.0 / (2 * self.cfg.n_layer) ** 0.5)

    def forward(self, ids: torch.Tensor, kv_caches=None, pos0: int = 0) -> torch.Tensor:
        delta, residual = self.wte(ids, pos0), None
        for i, blk in enumerate(self.blocks):
            cache = kv_caches[i] if kv_caches is not None else None
            if self.gradient_checkpointing and self.training and cache is None:
                if residual is None:
                    delta, residual = checkpoint(lambda d, b=blk: b(d), delta)
                else:
                    delta, residual = checkpoint(blk, delta, residual)
            else:
                delta, residual = blk(delta, residual, cache)
        h, _ = self.ln_f(delta, residual=residual)
        return h

    def create_kv_cache(self, batch: int, max_seq_len: int | None = None):
        from .attention import LayerKVCache
        p = next(self.parameters())
        return LayerKVCache(self.cfg.n_layer, batch, max_seq_len or self.cfg.n_ctx, self.cfg.n_head, self.cfg.head_dim(),
                            device=p.device, dtype=p.dtype)

    def forward_with_past(self, ids, past=None):
        """``(hidden states, cache)``: runs ``ids`` after whatever ``past`` (a cache from an earlier
        call, or ``None`` to start one) already holds."""
        ids = torch.as_tensor(ids).long()
        ids = ids.unsqueeze(0) if ids.dim() == 1 else ids
        if past is None:
            past = self.create_kv_cache(ids.shape[0])
        return self.forward(ids, past, past.seq_len()), past

    @classmethod
    def _config_from_json(cls, j):
        d = GPT2Config()
        return GPT2Config(vocab_size=int(j.get("vocab_size", d.vocab_size)), n_ctx=int(j.get("n_positions", j.get("n_ctx", d.n_ctx))),
                          n_embd=int(j.get("n_embd", d.n_embd)), n_layer=int(j.get("n_layer", d.n_layer)), n_head=int(j.get("n_head", d.n_head)),
                          layer_norm_eps=float(j.get("layer_norm_epsilon", d.layer_norm_eps)))


class GPT2LMHead(nn.Module, LoadStateDict, ModelApi, _Presets):
    ARCH = "gpt2"
    _config_from_json = GPT2._config_from_json

    """Language-model head tied to the token embedding (``lm_head.weight`` is ``wte``)."""

    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.transformer = GPT2(cfg, device, dtype)

    @classmethod
    def new(cls, cfg: GPT2Config): return cls(cfg)

    @property
    def lm_head_weight(self):
        return self.transformer.wte.wte.weight

    def gradient_checkpointing_enable(self, flag: bool = True):
        self.transformer.gradient_checkpointing = flag
        return self

    def forward_ids(self, ids, kv_caches=None, pos0: int = 0):
        """Logits over the padded vocabulary (``forward`` cuts them to ``vocab_size``)."""
        ids = torch.as_tensor(ids)
        ids = (ids.unsqueeze(0) if ids.dim() == 1 else ids).long()
        h = self.transformer(ids, kv_caches, pos0)
        return linear(h, self.lm_head_weight)

    def create_kv_cache(self, batch: int, max_seq_len: int | None = None):
        return self.transformer.create_kv_cache(batch, max_seq_len)

    def forward(self, ids, kv_caches=None, pos0: int = 0):
        return self.forward_ids(ids, kv_caches, pos0)[..., : self.cfg.vocab_size]

    def enable_context_parallel(self, process_group, form: str = "ulysses"):
        """Shards the sequence over ``process_group``: ``forward_with_loss`` then takes the whole
        sequence on every rank, runs this rank's slice (position embeddings offset accordingly;
        ``form``: "ulysses" all-to-all, "allgather" of K/V or "ring") and returns a loss whose mean over the
        ranks is the loss of the whole sequence."""
        from ..parallel.context_parallel import attention_fn
        attention_fn(form)                                   # validates the name
        self.cp_group = process_group
        for m in self.modules():
            if isinstance(m, CausalSelfAttention):
                m.cp_group, m.cp_form = process_group, form
        return self

    def forward_with_loss(self, ids, labels=None):
        """Shifted next-token cross-entropy: position t predicts token t+1 (gpt2.rs:182-266).
        Returns ``(loss, logits)`` where logits carry the padded vocabulary."""
        labels = ids if labels is None else labels
        cp = getattr(self, "cp_group", None)
        if cp is not None and cp.world_size() > 1:
            from ..parallel.context_parallel import shard_sequence
            tgt = torch.full_like(labels, -100)
            tgt[:, :-1] = labels[:, 1:]
            total = (tgt != -100).sum().clamp_min(1)
            local_ids = shard_sequence(ids, cp)
            logits = self.forward_ids(local_ids, pos0=cp.rank() * local_ids.shape[1])
            tl = shard_sequence(tgt, cp).reshape(-1)
            B, S, Vp = logits.shape
            scale = (tl != -100).sum() * cp.world_size() / total
            loss = L.cross_entropy(logits.view(B * S, Vp), tl, valid_classes=self.cfg.vocab_size) * scale
            return loss, logits
        logits = self.forward_ids(ids)
        B, S, Vp = logits.shape
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
        loss = L.cross_entropy(logits.view(B * S, Vp), tgt.view(-1), valid_classes=self.cfg.vocab_size)
        return loss, logits

    @torch.no_grad()
    def generate(self, ids, max_new_tokens: int = 20, temperature: float = 1.0, top_k=None, eos_token_id=None):
        from .generation import GenerationConfig, TextGenerator
        cfg = GenerationConfig(max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k,
                               do_sample=temperature != 1.0 or top_k is not None,
                               eos_token_ids=[eos_token_id] if eos_token_id is not None else [])
        return TextGenerator(cfg).generate(self, ids)
