"""Embedding layers of the language models.

Parity: crates/axonml-llm/src/embedding.rs (``TokenEmbedding`` with ``forward_ids``,
``PositionalEmbedding`` with ``forward_positions(seq_len, batch)``, ``SinusoidalPositionalEncoding``
with ``forward_seq`` -- angle = pos / 10000^(2i/d), sine in the even and cosine in the odd columns --,
``BertEmbedding`` = word + position + token-type embeddings, LayerNorm, dropout, with
``forward_with_ids(ids, token_type_ids, position_ids)``; ``GPT2Embedding`` lives in ``gpt2.py``).
Ids are integer tensors here (the reference carries them as u32 tensors)."""
from __future__ import annotations

import math

import torch

from .. import nn


class TokenEmbedding(nn.Module):
    def __init__(self, vocab_size: int, embed_dim: int, device=None, dtype=None):
        super().__init__()
        self.embedding = nn.Embedding(vocab_size, embed_dim, device=device, dtype=dtype)
        self.vocab_size, self.embed_dim = vocab_size, embed_dim

    @classmethod
    def new(cls, vocab_size: int, embed_dim: int): return cls(vocab_size, embed_dim)

    def forward_ids(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.embedding(input_ids.long())

    forward = forward_ids


class PositionalEmbedding(nn.Module):
    """Learned absolute positions 0 .. max_len-1."""

    def __init__(self, max_len: int, embed_dim: int, device=None, dtype=None):
        super().__init__()
        self.embedding = nn.Embedding(max_len, embed_dim, device=device, dtype=dtype)
        self.max_len, self.embed_dim = max_len, embed_dim

    @classmethod
    def new(cls, max_len: int, embed_dim: int): return cls(max_len, embed_dim)

    def forward_positions(self, seq_len: int, batch_size: int = 1, offset: int = 0) -> torch.Tensor:
        if offset + seq_len > self.max_len:
            from .error import InvalidInput
            raise InvalidInput(f"positions up to {offset + seq_len} exceed the table of {self.max_len}")
        pos = torch.arange(offset, offset + seq_len, device=self.embedding.weight.device)
        return self.embedding(pos).unsqueeze(0).expand(batch_size, seq_len, self.embed_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Positions for a [batch, seq, ...] tensor."""
        return self.forward_positions(x.shape[1], x.shape[0])


class SinusoidalPositionalEncoding(nn.Module):
    def __init__(self, max_len: int, embed_dim: int):
        super().__init__()
        pos = torch.arange(max_len, dtype=torch.float32).unsqueeze(1)
        i = torch.arange(embed_dim // 2, dtype=torch.float32)
        angle = pos / torch.pow(torch.tensor(10000.0), 2.0 * i / embed_dim)
        enc = torch.zeros(max_len, embed_dim)
        enc[:, 0:2 * (embed_dim // 2):2] = torch.sin(angle)
        enc[:, 1:2 * (embed_dim // 2):2] = torch.cos(angle)
        self.register_buffer("encodings", enc, persistent=False)
        self.max_len, self.embed_dim = max_len, embed_dim

    @classmethod
    def new(cls, max_len: int, embed_dim: int): return cls(max_len, embed_dim)

    def forward_seq(self, seq_len: int) -> torch.Tensor:
        return self.encodings[:seq_len]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x + encodings, for a [batch, seq, dim] tensor."""
        return x + self.encodings[:x.shape[1]].to(x.dtype)


class BertEmbedding(nn.Module):
    def __init__(self, vocab_size: int, max_position_embeddings: int, type_vocab_size: int, hidden_size: int,
                 layer_norm_eps: float = 1e-12, dropout_prob: float = 0.1):
        super().__init__()
        self.word_embeddings = nn.Embedding(vocab_size, hidden_size)
        self.position_embeddings = nn.Embedding(max_position_embeddings, hidden_size)
        self.token_type_embeddings = nn.Embedding(type_vocab_size, hidden_size)
        self.layer_norm = nn.LayerNorm(hidden_size, layer_norm_eps)
        self.dropout = nn.Dropout(dropout_prob)
        self.embed_dim = hidden_size

    @classmethod
    def new(cls, *a, **kw): return cls(*a, **kw)

    def forward_with_ids(self, input_ids, token_type_ids=None, position_ids=None) -> torch.Tensor:
        B, S = input_ids.shape
        if position_ids is None:
            position_ids = torch.arange(S, device=input_ids.device).unsqueeze(0).expand(B, S)
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(input_ids)
        e = (self.word_embeddings(input_ids.long()) + self.position_embeddings(position_ids.long())
             + self.token_type_embeddings(token_type_ids.long()))
        return self.dropout(self.layer_norm(e))

    forward = forward_with_ids


def scaled_embedding_init(weight: torch.Tensor, std: float | None = None) -> None:
    """N(0, std) initialisation, std = 1/sqrt(dim) when not given."""
    with torch.no_grad():
        weight.normal_(0.0, std if std is not None else 1.0 / math.sqrt(weight.shape[-1]))
