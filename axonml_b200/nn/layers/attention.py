"""MultiHeadAttention (crates/axonml-nn/src/layers/attention.rs:36-270): four Linear(E,E)
projections named ``q_proj, k_proj, v_proj, out_proj``; ``attention(q,k,v,mask)`` where
``mask == 0`` positions are excluded; ``forward(x)`` is self-attention.  The score/softmax/value
product runs through ``ops.attention.sdpa`` (flash-attention kernel on B200)."""
from __future__ import annotations

import torch

from ...ops.attention import sdpa
from ..module import Module
from .dropout import Dropout
from .linear import Linear


class MultiHeadAttention(Module):
    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, batch_first: bool = True):
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.batch_first = batch_first
        self.q_proj = Linear(embed_dim, embed_dim)
        self.k_proj = Linear(embed_dim, embed_dim)
        self.v_proj = Linear(embed_dim, embed_dim)
        self.out_proj = Linear(embed_dim, embed_dim)
        self.dropout = Dropout(dropout)

    @classmethod
    def new(cls, embed_dim, num_heads): return cls(embed_dim, num_heads)

    @classmethod
    def with_options(cls, embed_dim, num_heads, dropout, batch_first=True):
        return cls(embed_dim, num_heads, dropout, batch_first)

    def attention(self, query, key, value, mask=None, is_causal: bool = False):
        if not self.batch_first:
            query, key, value = (t.transpose(0, 1) for t in (query, key, value))
        B, Sq, _ = query.shape
        Sk = key.shape[1]
        q = self.q_proj(query).view(B, Sq, self.num_heads, self.head_dim)
        k = self.k_proj(key).view(B, Sk, self.num_heads, self.head_dim)
        v = self.v_proj(value).view(B, Sk, self.num_heads, self.head_dim)
        o = sdpa(q, k, v, mask=mask, causal=is_causal)
        o = self.dropout(o.reshape(B, Sq, self.embed_dim))
        out = self.out_proj(o)
        return out if self.batch_first else out.transpose(0, 1)

    def forward(self, x, mask=None):
        return self.attention(x, x, x, mask)
