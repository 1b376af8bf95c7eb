"""Flash attention on tcgen05 (``csrc/kernels/flash_fwd.cu``, ``flash_bwd.cu``): bf16,
head_dim 128, causal or full, grouped-query heads, token-major ``[B, S, H, D]`` tensors."""
from __future__ import annotations

import math

import torch

from .. import _native as N


def supported(q, k, v, mask, dropout_p) -> bool:
    if mask is not None or dropout_p > 0.0 or not N.is_blackwell():
        return False
    if not (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16):
        return False
    if q.dim() != 4 or q.shape[-1] != 128 or q.shape[2] % k.shape[2] != 0:
        return False
    return _HAVE_BWD or not (q.requires_grad or k.requires_grad or v.requires_grad)


def _strides(t):
    """(tensor, row_stride, batch_stride) with a layout the kernels accept: last dim contiguous,
    heads ``D`` apart, 16-byte aligned rows."""
    B, S, H, D = t.shape
    if (t.stride(3) != 1 or t.stride(2) != D or t.stride(1) % 8 or t.stride(0) % 8
            or t.data_ptr() % 16):
        t = t.contiguous()
    return t, t.stride(1), t.stride(0)


def set_one_tile(flag: bool) -> None:
    """Forces the forward kernel with one 128-query tile per CTA (``True``) instead of the choice by
    sequence length; for comparisons of the two kernels."""
    N.cuda().ax_flash_fwd_set_one_tile(int(bool(flag)))


def flash_fwd(q, k, v, causal: bool, scale: float | None = None):
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    q, qr, qb = _strides(q)
    k, kr, kb = _strides(k)
    v, vr, vb = _strides(v)
    out = torch.empty((B, Sq, Hq, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    rc = N.cuda().ax_flash_fwd(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(lse), B, Sq, Skv, Hq, Hkv,
                               D, N.c_int64(qr), N.c_int64(qb), N.c_int64(kr), N.c_int64(kb),
                               N.c_int64(vr), N.c_int64(vb), N.c_int64(out.stride(1)),
                               N.c_int64(out.stride(0)), int(causal), N.c_float(scale),
                               N.ptr(N.status_word(q.device)), N.stream_ptr())
    N.check(rc, "ax_flash_fwd")
    return out, lse, (q, k, v)


_HAVE_BWD = False


def flash_attention(q, k, v, causal: bool = False, scale: float | None = None):
    return flash_fwd(q, k, v, causal, scale)[0]


def flash_bwd(q, k, v, out, dout, lse, causal, scale, dq, dk, dv):
    """Writes dq/dk/dv (token-major views, any row/batch strides)."""
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    dout, dor, dob = _strides(dout)
    delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    assert dk.stride(1) == dv.stride(1) and dk.stride(0) == dv.stride(0)
    L = N.c_int64
    rc = N.cuda().ax_flash_bwd(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(dout), N.ptr(lse), N.ptr(delta), N.ptr(dq),
        N.ptr(dk), N.ptr(dv), B, Sq, Skv, Hq, Hkv, D, L(q.stride(1)), L(q.stride(0)), L(k.stride(1)),
        L(k.stride(0)), L(v.stride(1)), L(v.stride(0)), L(out.stride(1)), L(out.stride(0)), L(dor),
        L(dob), L(dq.stride(1)), L(dq.stride(0)), L(dk.stride(1)), L(dk.stride(0)), int(causal),
        N.c_float(scale), N.ptr(N.status_word(q.device)), N.stream_ptr())
    N.check(rc, "ax_flash_bwd")


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        out, lse, (q, k, v) = flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        flash_bwd(q, k, v, out, dout, lse, ctx.causal, ctx.scale, dq, dk, dv)
        return dq, dk, dv, None, None


class _FlashPackedFn(torch.autograd.Function):
    """Attention on a packed ``[B, S, Hq + 2*Hkv, D]`` tensor (q heads | k heads | v heads): the
    backward writes dq, dk, dv straight into one packed gradient tensor."""

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, causal, scale):
        scale = scale if scale is not None else 1.0 / math.sqrt(qkv.shape[-1])
        if not qkv.is_contiguous():
            qkv = qkv.contiguous()
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        out, lse, _ = flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (Hq, Hkv, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        Hq, Hkv, causal, scale = ctx.meta
        d = torch.empty_like(qkv)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        flash_bwd(q, k, v, out, dout, lse, causal, scale, d[:, :, :Hq], d[:, :, Hq:Hq + Hkv],
                  d[:, :, Hq + Hkv:])
        return d, None, None, None, None


_HAVE_BWD = True


def flash_attention(q, k, v, causal: bool = False, scale: float | None = None):  # noqa: F811
    return _FlashFn.apply(q, k, v, causal, scale)


def flash_attention_packed(qkv, Hq: int, Hkv: int, causal: bool = True, scale: float | None = None):
    return _FlashPackedFn.apply(qkv, Hq, Hkv, causal, scale)


def packed_supported(qkv) -> bool:
    return (N.is_blackwell() and qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 4
            and qkv.shape[-1] == 128)
