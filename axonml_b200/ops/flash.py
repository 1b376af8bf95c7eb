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
