"""Scaled-dot-product attention entry point.

``sdpa(q, k, v)`` takes token-major ``[B, S, H, D]`` tensors (the layout the fused QKV GEMM
produces), supports grouped-query attention (fewer K/V heads than Q heads), a causal flag or an
explicit mask.  bf16 inputs with head_dim 128 (or 64) on a B200 run the hand-written tcgen05
flash-attention kernels (forward and backward); everything else evaluates the same maths with
torch ops.

Parity: crates/axonml-llm/src/attention.rs:677-1005 (FlashAttention /
scaled_dot_product_attention), crates/axonml-nn/src/layers/attention.rs:125-217."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _flash_ok(q, k, v, mask, dropout_p) -> bool:
    from . import flash
    return flash.supported(q, k, v, mask, dropout_p)


def sdpa_reference(q, k, v, mask=None, causal: bool = False, scale: float | None = None):
    """Reference in fp32 (fp64 for fp64 inputs): q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] -> [B,Sq,Hq,D]."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cd = torch.float64 if q.dtype == torch.float64 else torch.float32      # never below the input's precision
    qf = q.to(cd).permute(0, 2, 1, 3)
    kf = k.to(cd).permute(0, 2, 1, 3)
    vf = v.to(cd).permute(0, 2, 1, 3)
    if Hkv != Hq:
        rep = Hq // Hkv
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        cm = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril(Sk - Sq)
        s = s.masked_fill(~cm, float("-inf"))
    if mask is not None:
        m = mask
        if m.dtype != torch.bool:
            m = m != 0
        while m.dim() < 4:
            m = m.unsqueeze(0)
        s = s.masked_fill(~m, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


def sdpa(q, k, v, mask=None, causal: bool = False, scale: float | None = None,
         dropout_p: float = 0.0):
    if _flash_ok(q, k, v, mask, dropout_p):
        from . import flash
        return flash.flash_attention(q, k, v, causal=causal, scale=scale)
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    if q.is_cuda and mask is None:
        qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        Sk = k.shape[1]
        attn_mask = None
        is_causal = causal
        if causal and Sq != Sk:
            # The causal mask of this package is aligned to the END of the key sequence (query i
            # sees keys up to i + Sk - Sq: what a KV cache and a key slice need); torch's
            # ``is_causal`` aligns to the start, so the mask is passed explicitly.
            is_causal = False
            if Sq > 1:
                attn_mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril(Sk - Sq)
        o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=attn_mask, is_causal=is_causal,
                                           scale=scale, dropout_p=dropout_p, enable_gqa=(Hkv != Hq))
        return o.permute(0, 2, 1, 3)
    o = sdpa_reference(q, k, v, mask, causal, scale)
    if dropout_p > 0:
        o = F.dropout(o, dropout_p)
    return o


def sdpa_packed(qkv, Hq: int, Hkv: int, causal: bool = True, scale: float | None = None,
                dropout_p: float = 0.0):
    """Self-attention on a packed ``[B, S, Hq + 2*Hkv, D]`` tensor laid out q heads | k heads |
    v heads (what a fused QKV projection produces).  On a B200 the flash kernels read the three
    parts in place and the backward writes one packed gradient."""
    from . import flash
    if dropout_p == 0.0 and flash.packed_supported(qkv):
        return flash.flash_attention_packed(qkv, Hq, Hkv, causal, scale)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    return sdpa(q, k, v, causal=causal, scale=scale, dropout_p=dropout_p)
