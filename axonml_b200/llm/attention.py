"""KV caches and attention helpers of the LLM crate (crates/axonml-llm/src/attention.rs:19-126,
:677-1005).  ``KVCache`` preallocates ``max_seq_len`` slots and appends in place (the reference
re-concatenates on every token, attention.rs:61-67); tensors are token-major ``[B, S, H, D]``."""
from __future__ import annotations

import dataclasses

import torch

from ..ops.attention import sdpa


class KVCache:
    def __init__(self, batch: int, max_seq_len: int, num_heads: int, head_dim: int, device=None,
                 dtype=torch.float32):
        self.key = torch.zeros(batch, max_seq_len, num_heads, head_dim, device=device, dtype=dtype)
        self.value = torch.zeros_like(self.key)
        self.seq_len = 0
        self.max_seq_len = max_seq_len

    @classmethod
    def new(cls, batch, max_seq_len, num_heads, head_dim, **kw): return cls(batch, max_seq_len, num_heads, head_dim, **kw)

    def update(self, k: torch.Tensor, v: torch.Tensor):
        """Appends ``k, v [B, S_new, H, D]``; returns views of everything cached so far."""
        n = k.shape[1]
        if self.seq_len + n > self.max_seq_len:
            raise ValueError("KV cache overflow")
        if self.key.dtype != k.dtype or self.key.device != k.device:
            self.key = self.key.to(device=k.device, dtype=k.dtype)
            self.value = self.value.to(device=v.device, dtype=v.dtype)
        self.key[:, self.seq_len:self.seq_len + n] = k
        self.value[:, self.seq_len:self.seq_len + n] = v
        self.seq_len += n
        return self.key[:, :self.seq_len], self.value[:, :self.seq_len]

    def len(self) -> int: return self.seq_len
    def __len__(self) -> int: return self.seq_len
    def is_empty(self) -> bool: return self.seq_len == 0
    def clear(self) -> None: self.seq_len = 0


class LayerKVCache:
    def __init__(self, num_layers: int, batch: int, max_seq_len: int, num_heads: int, head_dim: int,
                 device=None, dtype=torch.float32):
        self.layers = [KVCache(batch, max_seq_len, num_heads, head_dim, device, dtype) for _ in range(num_layers)]

    @classmethod
    def new(cls, *a, **kw): return cls(*a, **kw)

    def get_mut(self, i: int) -> KVCache: return self.layers[i]
    def __getitem__(self, i: int) -> KVCache: return self.layers[i]
    def seq_len(self) -> int: return self.layers[0].seq_len if self.layers else 0
    def clear(self) -> None:
        for c in self.layers:
            c.clear()


@dataclasses.dataclass
class FlashAttentionConfig:
    """Parity: crates/axonml-llm/src/attention.rs:636-660.  The block sizes are accepted for
    compatibility; the GPU kernel tiles 128 queries x 128 keys on its own."""
    block_size_q: int = 64
    block_size_kv: int = 64
    causal: bool = True
    softmax_scale: float | None = None
    dropout_p: float = 0.0


class FlashAttention:
    """Blockwise attention with online softmax (attention.rs:677-977).  Inputs ``[B, H, S, D]`` as
    in the reference; on a B200 (bf16, head_dim 64/128) this is the tcgen05 flash kernel."""

    def __init__(self, num_heads: int, dropout_p: float = 0.0, causal: bool = False, block_size: int = 64):
        self.num_heads, self.dropout_p, self.causal, self.block_size = num_heads, dropout_p, causal, block_size

    @classmethod
    def new(cls, num_heads, dropout_p=0.0, causal=False): return cls(num_heads, dropout_p, causal)

    def with_block_size(self, block_size: int):
        self.block_size = block_size
        return self

    def forward_qkv(self, q, k, v, scale=None):
        o = sdpa(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=self.causal, scale=scale)
        return o.transpose(1, 2)

    def memory_estimate(self, batch: int, seq_len: int, head_dim: int, bytes_per_el: int = 2) -> dict:
        std = batch * self.num_heads * seq_len * seq_len * bytes_per_el
        flash = batch * self.num_heads * seq_len * (head_dim + 2) * 4
        return {"standard_bytes": std, "flash_bytes": flash, "ratio": std / max(flash, 1)}


def scaled_dot_product_attention(q, k, v, mask=None, dropout_p: float = 0.0, is_causal: bool = False, scale=None):
    """``[B, H, S, D]`` API of attention.rs:982-1005."""
    o = sdpa(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), mask=mask, causal=is_causal,
             scale=scale, dropout_p=dropout_p)
    return o.transpose(1, 2)
