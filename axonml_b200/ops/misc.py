"""Embedding, rotary embedding, cast and transpose kernels (``csrc/kernels/misc.cu``)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N


def _dt(t):
    return 1 if t.dtype == torch.bfloat16 else 0


def _ok(t):
    return t.is_cuda and N.have_gpu() and t.dtype in (torch.float32, torch.bfloat16)


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, W, P, seq_len, pos0, padding_idx):
        ids = idx.reshape(-1).to(torch.int64).contiguous()
        T, D = ids.numel(), W.shape[1]
        out = torch.empty((T, D), dtype=W.dtype, device=W.device)
        N.check(N.cuda().ax_embedding_fwd(_dt(W), N.ptr(ids), N.ptr(W), N.ptr(P), N.ptr(out),
                                          N.c_int64(T), D, seq_len, pos0, N.c_int64(W.shape[0]),
                                          N.c_int64(padding_idx), N.stream_ptr()), "ax_embedding_fwd")
        ctx.save_for_backward(ids)
        ctx.meta = (W.shape, None if P is None else P.shape, W.dtype, seq_len, pos0, padding_idx)
        return out.view(*idx.shape, D)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        wshape, pshape, dtype, seq_len, pos0, padding_idx = ctx.meta
        D = wshape[1]
        d2 = dout.reshape(-1, D).contiguous()
        dW = torch.zeros(wshape, dtype=torch.float32, device=dout.device)
        dP = torch.zeros(pshape, dtype=torch.float32, device=dout.device) if pshape else None
        N.check(N.cuda().ax_embedding_bwd(_dt(d2), N.ptr(ids), N.ptr(d2), N.ptr(dW), N.ptr(dP),
                                          N.c_int64(ids.numel()), D, seq_len, pos0,
                                          N.c_int64(wshape[0]), N.c_int64(padding_idx),
                                          N.stream_ptr()), "ax_embedding_bwd")
        return None, dW.to(dtype), (dP.to(dtype) if dP is not None else None), None, None, None


def embedding(idx, weight, *, pos_weight=None, seq_len: int = 1, pos0: int = 0,
              padding_idx: int = -1):
    """``weight[idx]`` (+ ``pos_weight[pos0 + t % seq_len]`` for token t when given)."""
    if _ok(weight) and idx.is_cuda and (pos_weight is None or pos_weight.dtype == weight.dtype):
        return _EmbeddingFn.apply(idx, weight.contiguous(),
                                  None if pos_weight is None else pos_weight.contiguous(),
                                  seq_len, pos0, padding_idx)
    neg = idx < 0                     # negative ids give zero rows (vocabulary-parallel tables)
    out = F.embedding(idx.long().clamp_min(0), weight, padding_idx=None if padding_idx < 0 else padding_idx)
    out = out.masked_fill(neg.unsqueeze(-1), 0)
    if pos_weight is not None:
        pos = (torch.arange(idx.numel(), device=idx.device) % seq_len + pos0).view(idx.shape)
        out = out + F.embedding(pos, pos_weight)
    return out


def rope_tables(max_pos: int, head_dim: int, theta: float = 10000.0, device=None):
    """fp32 cos/sin tables ``[max_pos, head_dim/2]`` (half-split convention)."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64, device=device) / half))
    ang = torch.arange(max_pos, dtype=torch.float64, device=device)[:, None] * inv[None, :]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, seq_len, pos0, rot_heads=-1):
        out = _rope_launch(x, cos, sin, seq_len, pos0, 1.0, rot_heads)
        ctx.save_for_backward(cos, sin)
        ctx.meta = (seq_len, pos0, rot_heads)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _rope_launch(dy, cos, sin, ctx.meta[0], ctx.meta[1], -1.0, ctx.meta[2]), None, None, None, None, None


def _rope_launch(x, cos, sin, seq_len, pos0, sign, rot_heads=-1, positions=None):
    # x: [..., heads, head_dim] with token-major leading dims
    heads, hd = x.shape[-2], x.shape[-1]
    x3 = x.reshape(-1, heads, hd)
    if x3.stride(2) != 1 or x3.stride(1) != hd:
        x3 = x3.contiguous()
    out = torch.empty((x3.shape[0], heads, hd), dtype=x.dtype, device=x.device)
    N.check(N.cuda().ax_rope(_dt(x3), N.ptr(x3), N.ptr(out), N.ptr(cos), N.ptr(sin),
                             N.c_int64(x3.shape[0]), heads, hd, N.c_int64(x3.stride(0)),
                             N.c_int64(out.stride(0)), seq_len, pos0, N.c_float(sign),
                             heads if rot_heads < 0 else rot_heads, N.ptr(positions), N.stream_ptr()), "ax_rope")
    return out.view(x.shape)


def rope(x, cos, sin, *, seq_len: int, pos0: int = 0, rot_heads: int = -1):
    """Rotary embedding (half-split) of ``x[B*S or B,S, heads, head_dim]``; token t of the
    flattened leading dims has position ``pos0 + t % seq_len``.  With ``rot_heads >= 0`` only the
    first ``rot_heads`` heads are rotated and the rest are copied (packed q|k|v tensors)."""
    if _ok(x):
        return _RopeFn.apply(x, cos, sin, seq_len, pos0, rot_heads)
    if rot_heads >= 0 and rot_heads < x.shape[-2]:
        a = rope(x[..., :rot_heads, :], cos, sin, seq_len=seq_len, pos0=pos0)
        return torch.cat([a, x[..., rot_heads:, :]], dim=-2)
    hd = x.shape[-1]
    half = hd // 2
    lead = x.shape[:-2]
    T = 1
    for s in lead:
        T *= s
    pos = (torch.arange(T, device=x.device) % seq_len + pos0)
    c = cos[pos].view(*lead, 1, half).to(torch.float32)
    s = sin[pos].view(*lead, 1, half).to(torch.float32)
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


def rope_positions(x, cos, sin, positions, rot_heads: int = -1):
    """Rotary embedding with an explicit int32 position per token (decode batches where every
    sequence is at a different position).  ``x``: ``[T, heads, head_dim]``; inference only."""
    if _ok(x):
        return _rope_launch(x, cos, sin, 1, 0, 1.0, rot_heads, positions.to(torch.int32))
    hd = x.shape[-1]
    half = hd // 2
    nrot = x.shape[-2] if rot_heads < 0 else rot_heads
    c = cos[positions.long()].view(-1, 1, half).float()
    s = sin[positions.long()].view(-1, 1, half).float()
    a, b = x[:, :nrot, :half].float(), x[:, :nrot, half:].float()
    rot = torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)
    return torch.cat([rot, x[:, nrot:]], dim=1)


def cast(x: torch.Tensor, dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    kinds = {(torch.float32, torch.bfloat16): 0, (torch.bfloat16, torch.float32): 1,
             (torch.float32, torch.float32): 2, (torch.bfloat16, torch.bfloat16): 3}
    key = (x.dtype, dtype)
    if not (x.is_cuda and N.have_gpu() and key in kinds):
        return (x.float() * scale).to(dtype) if scale != 1.0 else x.to(dtype)
    x = x.contiguous()
    y = torch.empty(x.shape, dtype=dtype, device=x.device)
    N.check(N.cuda().ax_cast(kinds[key], N.ptr(x), N.ptr(y), N.c_int64(x.numel()), N.c_float(scale),
                             N.stream_ptr()), "ax_cast")
    return y


def transpose2d(x: torch.Tensor) -> torch.Tensor:
    if not (_ok(x) and x.dim() == 2):
        return x.t().contiguous()
    x = x.contiguous()
    y = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
    N.check(N.cuda().ax_transpose(_dt(x), N.ptr(x), N.ptr(y), x.shape[0], x.shape[1],
                                  N.stream_ptr()), "ax_transpose")
    return y
