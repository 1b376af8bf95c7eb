"""LayerNorm / RMSNorm on the hand-written kernels (``csrc/kernels/norm.cu``), with an optional
fused residual add.  Falls back to torch maths on CPU.

Parity: crates/axonml-nn/src/layers/norm.rs:413-482 (LayerNorm), crates/axonml-llm/src/llama.rs:138-198
(RMSNorm)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N


def _dt(t):
    return 1 if t.dtype == torch.bfloat16 else 0


def _kernel_ok(x, w):
    if not (x.is_cuda and N.have_gpu()):
        return False
    if x.shape[-1] % 8 != 0:
        return False
    pair = (x.dtype, w.dtype)
    return pair in ((torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                    (torch.float32, torch.float32))


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, b, eps, rms):
        D = x.shape[-1]
        x2 = x.reshape(-1, D).contiguous()
        r2 = residual.reshape(-1, D).contiguous() if residual is not None else None
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if r2 is not None else None
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        N.check(N.cuda().ax_norm_fwd(int(rms), _dt(x2), _dt(w), N.ptr(x2), N.ptr(r2), N.ptr(w),
                                     N.ptr(b), N.ptr(y), N.ptr(h), N.ptr(mean), N.ptr(rstd), rows, D,
                                     N.c_float(eps), N.stream_ptr()), "ax_norm_fwd")
        ctx.save_for_backward(h if h is not None else x2, w, mean, rstd)
        ctx.rms, ctx.has_bias, ctx.has_res, ctx.shape = rms, b is not None, r2 is not None, x.shape
        if h is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        xin, w, mean, rstd = ctx.saved_tensors
        rows, D = xin.shape
        dy2 = dy.reshape(rows, D).contiguous()
        dres = dh.reshape(rows, D).contiguous() if (ctx.has_res and dh is not None) else None
        dx = torch.empty_like(xin)
        groups = N.cuda().ax_norm_bwd_groups(rows)
        scratch = torch.empty(groups * 2 * D, dtype=torch.float32, device=xin.device)
        dw = torch.empty_like(w)
        db = torch.empty_like(w) if ctx.has_bias else None
        N.check(N.cuda().ax_norm_bwd(int(ctx.rms), _dt(xin), _dt(w), N.ptr(dy2), N.ptr(xin),
                                     N.ptr(w), N.ptr(mean), N.ptr(rstd), N.ptr(dres), N.ptr(dx),
                                     N.ptr(dw), N.ptr(db), N.ptr(scratch), groups, rows, D,
                                     N.stream_ptr()), "ax_norm_bwd")
        dxv = dx.view(ctx.shape)
        return dxv, (dxv if ctx.has_res else None), dw, db, None, None


def _ref(x, residual, w, b, eps, rms):
    h = x if residual is None else x + residual
    cd = torch.float64 if h.dtype == torch.float64 else torch.float32     # never below the input's precision
    hf = h.to(cd)
    if rms:
        y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w.to(cd)
    else:
        y = F.layer_norm(hf, (h.shape[-1],), w.to(cd), None if b is None else b.to(cd), eps)
    y = y.to(x.dtype)
    return (y, h) if residual is not None else (y, None)


def layer_norm(x, weight, bias=None, eps: float = 1e-5, residual=None):
    """LayerNorm over the last dim.  With ``residual`` returns ``(norm(x+residual), x+residual)``."""
    if _kernel_ok(x, weight):
        y, h = _NormFn.apply(x, residual, weight, bias, eps, False)
    else:
        y, h = _ref(x, residual, weight, bias, eps, False)
    return (y, h) if residual is not None else y


def rms_norm(x, weight, eps: float = 1e-5, residual=None):
    """RMSNorm over the last dim (``x * rsqrt(mean(x^2)+eps) * weight``)."""
    if _kernel_ok(x, weight):
        y, h = _NormFn.apply(x, residual, weight, None, eps, True)
    else:
        y, h = _ref(x, residual, weight, None, eps, True)
    return (y, h) if residual is not None else y
