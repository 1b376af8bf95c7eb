"""Generic transformer encoder / decoder stacks of the language-model package.

Parity: crates/axonml-llm/src/attention.rs:130-260 (``MultiHeadSelfAttention`` with ``query``,
``key``, ``value``, ``out_proj`` and ``forward_with_mask``: an additive mask, 0 to attend and -inf
to hide), crates/axonml-llm/src/transformer.rs (``FeedForward`` fc1 -> activation -> fc2 -> dropout
with the activation chosen by name, ``TransformerEncoderBlock`` in pre-norm or post-norm order,
``TransformerDecoderBlock`` = pre-norm causal block, ``TransformerEncoder(num_layers, hidden, heads,
intermediate, dropout, eps, activation, pre_norm)`` with ``forward_with_mask``,
``TransformerDecoder(num_layers, n_embd, n_head, max_seq_len, dropout, eps, activation)`` ending in
``ln_f``) and config.rs:9-45 (``TransformerConfig``).  Without a mask the attention runs on the
flash kernel (bf16/fp16 on the GPU) through ``ops.attention.sdpa``; the activation is fused into
the first feed-forward GEMM."""
from __future__ import annotations

import dataclasses
import math

import torch

from .. import nn
from ..ops.attention import sdpa

_ACT = {"gelu": "gelu", "relu": "relu", "silu": "silu", "swish": "silu", "tanh": "tanh"}


@dataclasses.dataclass
class TransformerConfig:
    hidden_size: int = 768
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    num_layers: int = 12
    max_position_embeddings: int = 512
    vocab_size: int = 30522
    dropout_prob: float = 0.1
    attention_dropout_prob: float = 0.1
    layer_norm_eps: float = 1e-12
    activation: str = "gelu"

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def validate(self) -> None:
        from .error import InvalidConfig
        if self.hidden_size % self.num_attention_heads:
            raise InvalidConfig(f"hidden_size {self.hidden_size} is not divisible by {self.num_attention_heads} heads")
        if self.activation not in _ACT:
            raise InvalidConfig(f"unknown activation {self.activation!r}")


class MultiHeadSelfAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, dropout: float = 0.0, device=None, dtype=None):
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError("hidden_size must be divisible by num_heads")
        kw = dict(device=device, dtype=dtype)
        self.query, self.key = nn.Linear(hidden_size, hidden_size, **kw), nn.Linear(hidden_size, hidden_size, **kw)
        self.value, self.out_proj = nn.Linear(hidden_size, hidden_size, **kw), nn.Linear(hidden_size, hidden_size, **kw)
        self.attn_dropout = nn.Dropout(dropout)
        self.num_heads, self.head_dim = num_heads, hidden_size // num_heads
        self.scale = 1.0 / math.sqrt(self.head_dim)

    @classmethod
    def new(cls, hidden_size: int, num_heads: int, dropout: float = 0.0): return cls(hidden_size, num_heads, dropout)

    def forward_with_mask(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor | None = None, causal: bool = False):
        """``attention_mask``: a floating tensor is added to the scores (0 attends, -inf hides); a
        boolean tensor attends where True.  It broadcasts against [batch, heads, query, key]; a
        [batch, key] tensor is taken as a per-key padding mask."""
        B, S, H = hidden_states.shape
        q = self.query(hidden_states).view(B, S, self.num_heads, self.head_dim)
        k = self.key(hidden_states).view(B, S, self.num_heads, self.head_dim)
        v = self.value(hidden_states).view(B, S, self.num_heads, self.head_dim)
        p_drop = self.attn_dropout.p if self.training else 0.0
        if attention_mask is None and p_drop == 0.0:
            ctx = sdpa(q, k, v, causal=causal, scale=self.scale)
        else:
            scores = torch.matmul(q.permute(0, 2, 1, 3), k.permute(0, 2, 3, 1)) * self.scale      # [B, heads, S, S]
            if attention_mask is not None:
                m = attention_mask
                if m.dim() == 2 and m.shape == (B, S):
                    m = m[:, None, None, :]
                while m.dim() < 4:
                    m = m.unsqueeze(0)
                scores = scores.masked_fill(~m, float("-inf")) if m.dtype == torch.bool else scores + m.to(scores.dtype)
            if causal:
                scores = scores.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=scores.device).tril(), float("-inf"))
            probs = torch.nan_to_num(torch.softmax(scores.float(), dim=-1)).to(v.dtype)
            ctx = torch.matmul(self.attn_dropout(probs), v.permute(0, 2, 1, 3)).permute(0, 2, 1, 3)
        return self.out_proj(ctx.reshape(B, S, H))

    def forward(self, x):
        return self.forward_with_mask(x, None)


class FeedForward(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, dropout: float = 0.0, activation: str = "gelu", device=None, dtype=None):
        super().__init__()
        if activation not in _ACT:
            raise ValueError(f"unknown activation {activation!r}")
        self.fc1 = nn.Linear(hidden_size, intermediate_size, activation=_ACT[activation], device=device, dtype=dtype)
        self.fc2 = nn.Linear(intermediate_size, hidden_size, device=device, dtype=dtype)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        return self.dropout(self.fc2(self.fc1(x)))


class TransformerEncoderBlock(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, intermediate_size: int, dropout: float = 0.0, layer_norm_eps: float = 1e-12,
                 activation: str = "gelu", pre_norm: bool = False, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.attention = MultiHeadSelfAttention(hidden_size, num_heads, dropout, **kw)
        self.ln1 = nn.LayerNorm(hidden_size, layer_norm_eps, **kw)
        self.ffn = FeedForward(hidden_size, intermediate_size, dropout, activation, **kw)
        self.ln2 = nn.LayerNorm(hidden_size, layer_norm_eps, **kw)
        self.dropout = nn.Dropout(dropout)
        self.pre_norm = pre_norm

    def forward_with_mask(self, x, attention_mask=None):
        if self.pre_norm:
            x = x + self.dropout(self.attention.forward_with_mask(self.ln1(x), attention_mask))
            return x + self.dropout(self.ffn(self.ln2(x)))
        x = self.ln1(x + self.dropout(self.attention.forward_with_mask(x, attention_mask)))
        return self.ln2(x + self.dropout(self.ffn(x)))

    def forward(self, x):
        return self.forward_with_mask(x, None)


class TransformerDecoderBlock(nn.Module):
    """Pre-norm block with causal self-attention: x + attn(ln1 x), then x + ffn(ln2 x)."""

    def __init__(self, n_embd: int, n_head: int, max_seq_len: int, dropout: float = 0.0, layer_norm_eps: float = 1e-5,
                 activation: str = "gelu", device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.ln1 = nn.LayerNorm(n_embd, layer_norm_eps, **kw)
        self.attention = MultiHeadSelfAttention(n_embd, n_head, dropout, **kw)
        self.ln2 = nn.LayerNorm(n_embd, layer_norm_eps, **kw)
        self.ffn = FeedForward(n_embd, 4 * n_embd, dropout, activation, **kw)
        self.max_seq_len = max_seq_len

    def forward(self, x):
        if x.shape[1] > self.max_seq_len:
            from .error import InvalidInput
            raise InvalidInput(f"sequence of {x.shape[1]} tokens exceeds max_seq_len {self.max_seq_len}")
        x = x + self.attention.forward_with_mask(self.ln1(x), None, causal=True)
        return x + self.ffn(self.ln2(x))


class TransformerEncoder(nn.Module):
    def __init__(self, num_layers: int, hidden_size: int, num_heads: int, intermediate_size: int, dropout: float = 0.0,
                 layer_norm_eps: float = 1e-12, activation: str = "gelu", pre_norm: bool = False, device=None, dtype=None):
        super().__init__()
        self.layers = nn.ModuleList([TransformerEncoderBlock(hidden_size, num_heads, intermediate_size, dropout, layer_norm_eps,
                                                             activation, pre_norm, device=device, dtype=dtype)
                                     for _ in range(num_layers)])

    @classmethod
    def from_config(cls, cfg: TransformerConfig, pre_norm: bool = False):
        cfg.validate()
        return cls(cfg.num_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size, cfg.dropout_prob,
                   cfg.layer_norm_eps, cfg.activation, pre_norm)

    def forward_with_mask(self, x, attention_mask=None):
        for layer in self.layers:
            x = layer.forward_with_mask(x, attention_mask)
        return x

    def forward(self, x):
        return self.forward_with_mask(x, None)


class TransformerDecoder(nn.Module):
    def __init__(self, num_layers: int, n_embd: int, n_head: int, max_seq_len: int, dropout: float = 0.0,
                 layer_norm_eps: float = 1e-5, activation: str = "gelu", device=None, dtype=None):
        super().__init__()
        self.layers = nn.ModuleList([TransformerDecoderBlock(n_embd, n_head, max_seq_len, dropout, layer_norm_eps, activation,
                                                             device=device, dtype=dtype) for _ in range(num_layers)])
        self.ln_f = nn.LayerNorm(n_embd, layer_norm_eps, device=device, dtype=dtype)

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return self.ln_f(x)
