"""Fused cross-entropy and row softmax on ``csrc/kernels/softmax_ce.cu``.

The cross-entropy keeps only the per-row log-sum-exp between forward and backward; its backward
recomputes probabilities from the logits.  ``valid_classes`` lets the logits carry a padded
vocabulary (extra columns are ignored in the loss and get a zero gradient).

Parity: CrossEntropyLoss crates/axonml-nn/src/loss.rs:166-204 (made differentiable), softmax /
log_softmax crates/axonml-nn/src/functional.rs:85-120 (made dim-aware)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N


def _dt(t):
    return 1 if t.dtype == torch.bfloat16 else 0


def _ok(t):
    return t.is_cuda and N.have_gpu() and t.dtype in (torch.float32, torch.bfloat16)


class _CEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, valid_classes, ignore_index, reduction):
        Vpad = logits.shape[-1]
        l2 = logits.reshape(-1, Vpad)
        if l2.stride(1) != 1:
            l2 = l2.contiguous()
        t = target.reshape(-1).to(torch.int64).contiguous()
        rows = l2.shape[0]
        V = valid_classes or Vpad
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lib = N.cuda()
        N.check(lib.ax_ce_fwd(_dt(l2), N.ptr(l2), N.ptr(t), N.ptr(loss), N.ptr(lse), rows, V,
                              N.c_int64(l2.stride(0)), N.c_int64(ignore_index), N.stream_ptr()),
                "ax_ce_fwd")
        ctx.save_for_backward(l2, t, lse)
        ctx.V, ctx.Vpad, ctx.ignore_index, ctx.reduction = V, Vpad, ignore_index, reduction
        ctx.shape = logits.shape
        if reduction == "none":
            ctx.count = None
            return loss.view(target.shape)
        out = torch.empty(1, dtype=torch.float32, device=logits.device)
        if reduction == "sum":
            ctx.count = None
            N.check(lib.ax_reduce_sum_f32(N.ptr(loss), N.ptr(out), N.c_int64(rows), N.c_float(1.0),
                                          N.stream_ptr()), "ax_reduce_sum_f32")
            return out[0]
        cnt = torch.empty(1, dtype=torch.float32, device=logits.device)
        N.check(lib.ax_count_valid(N.ptr(t), N.ptr(cnt), N.c_int64(rows), N.c_int64(ignore_index), V,
                                   N.stream_ptr()), "ax_count_valid")
        N.check(lib.ax_reduce_sum_f32(N.ptr(loss), N.ptr(out), N.c_int64(rows), N.c_float(1.0),
                                      N.stream_ptr()), "ax_reduce_sum_f32")
        ctx.count = cnt
        return (out / cnt.clamp_min(1.0))[0]

    @staticmethod
    def backward(ctx, g):
        l2, t, lse = ctx.saved_tensors
        rows = l2.shape[0]
        dl = torch.empty_like(l2)
        g = g.to(torch.float32).contiguous()
        per_row = 0
        if ctx.reduction == "none":
            gs = g.reshape(-1)
            per_row = 1
        elif ctx.reduction == "mean":
            gs = (g / ctx.count.clamp_min(1.0)).reshape(1)
        else:
            gs = g.reshape(1)
        N.check(N.cuda().ax_ce_bwd(_dt(l2), N.ptr(l2), N.ptr(t), N.ptr(lse), N.ptr(gs), per_row,
                                   N.c_float(1.0), N.ptr(dl), rows, ctx.V, ctx.Vpad,
                                   N.c_int64(l2.stride(0)), N.c_int64(ctx.ignore_index),
                                   N.stream_ptr()), "ax_ce_bwd")
        return dl.view(ctx.shape), None, None, None, None


def cross_entropy(logits, target, *, valid_classes: int | None = None, ignore_index: int = -100,
                  reduction: str = "mean"):
    """Cross-entropy of ``logits[..., C]`` against class indices ``target[...]``."""
    if _ok(logits) and target.dtype in (torch.int64, torch.int32, torch.float32):
        return _CEFn.apply(logits, target, valid_classes, ignore_index, reduction)
    lg = logits if valid_classes is None else logits[..., :valid_classes]
    cd = torch.float64 if lg.dtype == torch.float64 else torch.float32      # never below the input's precision
    return F.cross_entropy(lg.reshape(-1, lg.shape[-1]).to(cd), target.reshape(-1).long(),
                           ignore_index=ignore_index, reduction=reduction).reshape(
                               target.shape if reduction == "none" else ())


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, log_mode):
        V = x.shape[-1]
        x2 = x.reshape(-1, V).contiguous()
        y = torch.empty_like(x2)
        N.check(N.cuda().ax_softmax_fwd(_dt(x2), N.ptr(x2), N.ptr(y), x2.shape[0], V, N.c_int64(V),
                                        int(log_mode), N.stream_ptr()), "ax_softmax_fwd")
        ctx.save_for_backward(y)
        ctx.log_mode, ctx.shape = log_mode, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        V = y.shape[-1]
        dy2 = dy.reshape(-1, V).contiguous()
        dx = torch.empty_like(y)
        N.check(N.cuda().ax_softmax_bwd(_dt(y), N.ptr(dy2), N.ptr(y), N.ptr(dx), y.shape[0], V,
                                        N.c_int64(V), int(ctx.log_mode), N.stream_ptr()),
                "ax_softmax_bwd")
        return dx.view(ctx.shape), None


def softmax(x, dim: int = -1, log: bool = False):
    """Dim-aware (log-)softmax; the kernel handles the last dim, other dims are moved there."""
    if not _ok(x):
        return F.log_softmax(x, dim) if log else F.softmax(x, dim)
    nd = x.dim()
    d = dim % nd
    if d != nd - 1:
        return _SoftmaxFn.apply(x.movedim(d, -1), log).movedim(-1, d)
    return _SoftmaxFn.apply(x, log)


def log_softmax(x, dim: int = -1):
    return softmax(x, dim, log=True)
