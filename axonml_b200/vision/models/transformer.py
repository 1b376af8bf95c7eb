"""Transformer encoder / decoder and VisionTransformer tiny/small/base/large
(crates/axonml-vision/src/models/transformer.rs)."""
from __future__ import annotations

import math

import torch

from ... import nn
from ...ops.attention import sdpa


class _MHA(nn.Module):
    def __init__(self, d_model: int, nhead: int, dropout: float = 0.0):
        super().__init__()
        self.h, self.hd = nhead, d_model // nhead
        self.q_proj, self.k_proj = nn.Linear(d_model, d_model), nn.Linear(d_model, d_model)
        self.v_proj, self.out_proj = nn.Linear(d_model, d_model), nn.Linear(d_model, d_model)

    def forward(self, q, k, v, causal=False, mask=None):
        """``mask``: attend where non-zero / True; broadcasts against [batch, heads, query, key]."""
        B, Sq, E = q.shape
        Sk = k.shape[1]
        o = sdpa(self.q_proj(q).view(B, Sq, self.h, self.hd), self.k_proj(k).view(B, Sk, self.h, self.hd),
                 self.v_proj(v).view(B, Sk, self.h, self.hd), mask=mask, causal=causal)
        return self.out_proj(o.reshape(B, Sq, E))


class PositionalEncoding(nn.Module):
    """Fixed sinusoidal position signal added to a [batch, seq, d_model] input
    (crates/axonml-vision/src/models/transformer.rs:29-90).  Column pairs (2k, 2k+1) share the
    frequency 10000^(-2k/d_model): sine in the even, cosine in the odd column.  (The reference
    gives every column its own exponent i/d_model, so its odd columns sit half a step off the
    usual table; the usual table is what is built here.)"""

    def __init__(self, d_model: int, max_len: int = 5000):
        super().__init__()
        pos = torch.arange(max_len, dtype=torch.float32).unsqueeze(1)
        k = torch.arange(0, d_model, 2, dtype=torch.float32)
        div = torch.exp(-(k / d_model) * math.log(10000.0))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div[: d_model // 2])
        self.register_buffer("encoding", pe, persistent=False)
        self.max_len, self.d_model = max_len, d_model

    @classmethod
    def new(cls, d_model: int, max_len: int): return cls(d_model, max_len)

    def forward(self, x):
        if x.shape[1] > self.max_len:
            raise ValueError(f"sequence of {x.shape[1]} exceeds max_len {self.max_len}")
        return x + self.encoding[: x.shape[1]].to(x.dtype)


class TransformerEncoderLayer(nn.Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1, activation: str = "gelu"):
        super().__init__()
        self.attn = _MHA(d_model, nhead, dropout)
        self.norm1, self.norm2 = nn.LayerNorm(d_model), nn.LayerNorm(d_model)
        self.fc1 = nn.Linear(d_model, dim_feedforward, activation=activation)
        self.fc2 = nn.Linear(dim_feedforward, d_model)
        self.drop = nn.Dropout(dropout)
        self._d_model = d_model

    def d_model(self) -> int: return self._d_model

    def forward_with_mask(self, x, src_mask=None):
        """The layer with an attention mask over the keys (non-zero = may be attended)."""
        h = self.norm1(x)
        x = x + self.drop(self.attn(h, h, h, mask=src_mask))
        return x + self.drop(self.fc2(self.fc1(self.norm2(x))))

    def forward(self, x):
        return self.forward_with_mask(x, None)


class TransformerDecoderLayer(nn.Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1):
        super().__init__()
        self.self_attn, self.cross_attn = _MHA(d_model, nhead), _MHA(d_model, nhead)
        self.norm1, self.norm2, self.norm3 = nn.LayerNorm(d_model), nn.LayerNorm(d_model), nn.LayerNorm(d_model)
        self.fc1 = nn.Linear(d_model, dim_feedforward, activation="gelu")
        self.fc2 = nn.Linear(dim_feedforward, d_model)
        self.drop = nn.Dropout(dropout)

    def forward_with_memory(self, x, memory, tgt_mask=None, memory_mask=None):
        """Decoder layer with explicit masks: ``tgt_mask`` over the target's own positions (causal
        when ``None``), ``memory_mask`` over the encoder output."""
        h = self.norm1(x)
        x = x + self.drop(self.self_attn(h, h, h, causal=tgt_mask is None, mask=tgt_mask))
        x = x + self.drop(self.cross_attn(self.norm2(x), memory, memory, mask=memory_mask))
        return x + self.drop(self.fc2(self.fc1(self.norm3(x))))

    def forward(self, x, memory):
        return self.forward_with_memory(x, memory)


class TransformerEncoder(nn.Module):
    def __init__(self, d_model, nhead, num_layers, dim_feedforward=2048, dropout=0.1):
        super().__init__()
        self.layers = nn.ModuleList([TransformerEncoderLayer(d_model, nhead, dim_feedforward, dropout) for _ in range(num_layers)])
        self.norm = nn.LayerNorm(d_model)

    def forward_with_mask(self, x, mask=None):
        for l in self.layers:
            x = l.forward_with_mask(x, mask)
        return self.norm(x)

    def forward(self, x):
        return self.forward_with_mask(x, None)


class TransformerDecoder(nn.Module):
    def __init__(self, d_model, nhead, num_layers, dim_feedforward=2048, dropout=0.1):
        super().__init__()
        self.layers = nn.ModuleList([TransformerDecoderLayer(d_model, nhead, dim_feedforward, dropout) for _ in range(num_layers)])
        self.norm = nn.LayerNorm(d_model)

    def forward_with_memory(self, x, memory, tgt_mask=None, memory_mask=None):
        for l in self.layers:
            x = l.forward_with_memory(x, memory, tgt_mask, memory_mask)
        return self.norm(x)

    def forward(self, x, memory):
        return self.forward_with_memory(x, memory)


class Transformer(nn.Module):
    def __init__(self, d_model=512, nhead=8, num_encoder_layers=6, num_decoder_layers=6, dim_feedforward=2048, dropout=0.1):
        super().__init__()
        self.encoder = TransformerEncoder(d_model, nhead, num_encoder_layers, dim_feedforward, dropout)
        self.decoder = TransformerDecoder(d_model, nhead, num_decoder_layers, dim_feedforward, dropout)

        self._d_model = d_model

    def d_model(self) -> int: return self._d_model

    def forward_full(self, src, tgt, src_mask=None, tgt_mask=None, memory_mask=None):
        """Encoder then decoder with every mask explicit (transformer.rs:482-493)."""
        memory = self.encoder.forward_with_mask(src, src_mask)
        return self.decoder.forward_with_memory(tgt, memory, tgt_mask, memory_mask)

    def forward(self, src, tgt): return self.forward_full(src, tgt)


class VisionTransformer(nn.Module):
    def __init__(self, image_size=224, patch_size=16, in_channels=3, num_classes=1000, d_model=768, depth=12,
                 nhead=12, mlp_ratio=4.0, dropout=0.0):
        super().__init__()
        self.patch_size = patch_size
        n = (image_size // patch_size) ** 2
        self.patch_embed = nn.Linear(in_channels * patch_size * patch_size, d_model)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, d_model))
        self.pos_embed = nn.Parameter(torch.randn(1, n + 1, d_model) * 0.02)
        self.encoder = TransformerEncoder(d_model, nhead, depth, int(d_model * mlp_ratio), dropout)
        self.head = nn.Linear(d_model, num_classes)

    @classmethod
    def vit_tiny(cls, image_size=224, num_classes=1000): return cls(image_size, 16, 3, num_classes, 192, 12, 3)
    @classmethod
    def vit_small(cls, image_size=224, num_classes=1000): return cls(image_size, 16, 3, num_classes, 384, 12, 6)
    @classmethod
    def vit_base(cls, image_size=224, num_classes=1000): return cls(image_size, 16, 3, num_classes, 768, 12, 12)
    @classmethod
    def vit_large(cls, image_size=224, num_classes=1000): return cls(image_size, 16, 3, num_classes, 1024, 24, 16)

    def forward(self, x):
        B, C, H, W = x.shape
        p = self.patch_size
        patches = x.unfold(2, p, p).unfold(3, p, p).permute(0, 2, 3, 1, 4, 5).reshape(B, -1, C * p * p)
        h = self.patch_embed(patches)
        h = torch.cat([self.cls_token.to(h.dtype).expand(B, -1, -1), h], 1) + self.pos_embed.to(h.dtype)
        return self.head(self.encoder(h)[:, 0])


def vit_base() -> VisionTransformer:
    """ViT-Base/16 for 224x224 inputs and 1000 classes (transformer.rs:754-756)."""
    return VisionTransformer.vit_base(224, 1000)


def vit_large() -> VisionTransformer:
    """ViT-Large/16 for 224x224 inputs and 1000 classes (transformer.rs:760-762)."""
    return VisionTransformer.vit_large(224, 1000)
