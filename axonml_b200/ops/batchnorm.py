"""BatchNorm2d and MaxPool2d on channels-last bf16 activations (``csrc/kernels/batchnorm_pool.cu``).

``batch_norm`` optionally fuses a residual add and a ReLU into the normalisation pass, which is what
a ResNet block needs after each convolution; the backward applies the ReLU mask from the saved
output and returns the residual's gradient too.  Running statistics follow the reference
(biased batch variance, ``running = (1-m)*running + m*batch``, norm.rs:339-357)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N


def _rows_cols(x):
    n, c, h, w = x.shape
    return n * h * w, c


def supported(x) -> bool:
    return (N.have_gpu() and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4
            and x.is_contiguous(memory_format=torch.channels_last) and x.shape[1] % 8 == 0 and 8 <= x.shape[1] <= 2048)


class _BNTrain(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, momentum, eps, relu, residual):
        R, C = _rows_cols(x)
        dev = x.device
        y = torch.empty_like(x)                         # keeps the channels-last strides
        stats = torch.zeros(6 * C, dtype=torch.float32, device=dev)
        sums, mean, rstd, scale, shift = stats[:2 * C], stats[2 * C:3 * C], stats[3 * C:4 * C], stats[4 * C:5 * C], stats[5 * C:]
        w = weight.detach().float().contiguous() if weight is not None else None
        b = bias.detach().float().contiguous() if bias is not None else None
        if residual is not None and not residual.is_contiguous(memory_format=torch.channels_last):
            residual = residual.contiguous(memory_format=torch.channels_last)
        rc = N.cuda().ax_batchnorm_fwd_train(N.ptr(x), N.ptr(residual), N.ptr(w), N.ptr(b), N.ptr(y), N.ptr(mean), N.ptr(rstd),
                                             N.ptr(scale), N.ptr(shift), N.ptr(running_mean), N.ptr(running_var), N.ptr(sums),
                                             N.c_int64(R), C, N.c_float(momentum), N.c_float(eps), int(relu), N.stream_ptr())
        N.check(rc, "ax_batchnorm_fwd_train")
        ctx.save_for_backward(x, y if relu else None, mean, rstd, scale)
        ctx.has_res, ctx.wdtype = residual is not None, (weight.dtype if weight is not None else None)
        ctx.bdtype = bias.dtype if bias is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, mean, rstd, scale = ctx.saved_tensors
        R, C = _rows_cols(x)
        if not dy.is_contiguous(memory_format=torch.channels_last):
            dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if ctx.has_res else None
        sums = torch.zeros(2 * C, dtype=torch.float32, device=x.device)
        rc = N.cuda().ax_batchnorm_bwd(N.ptr(dy), N.ptr(x), N.ptr(y), N.ptr(mean), N.ptr(rstd), N.ptr(scale), N.ptr(dx),
                                       N.ptr(dres), N.ptr(sums), N.c_int64(R), C, N.stream_ptr())
        N.check(rc, "ax_batchnorm_bwd")
        dw = sums[C:].to(ctx.wdtype) if ctx.wdtype is not None and ctx.needs_input_grad[1] else None
        db = sums[:C].to(ctx.bdtype) if ctx.bdtype is not None and ctx.needs_input_grad[2] else None
        return dx, dw, db, None, None, None, None, None, dres


def batch_norm(x, weight, bias, running_mean, running_var, training: bool, momentum: float, eps: float,
               relu: bool = False, residual=None):
    """``relu?(bn(x) + residual?)``.  In training mode the running statistics are updated in place."""
    if supported(x):
        if training:
            return _BNTrain.apply(x, weight, bias, running_mean, running_var, momentum, eps, relu, residual)
        if not torch.is_grad_enabled() or not (x.requires_grad or (weight is not None and weight.requires_grad)):
            R, C = _rows_cols(x)
            y = torch.empty_like(x)
            ss = torch.empty(2 * C, dtype=torch.float32, device=x.device)
            w = weight.detach().float().contiguous() if weight is not None else None
            b = bias.detach().float().contiguous() if bias is not None else None
            if residual is not None and not residual.is_contiguous(memory_format=torch.channels_last):
                residual = residual.contiguous(memory_format=torch.channels_last)
            rc = N.cuda().ax_batchnorm_fwd_eval(N.ptr(x), N.ptr(residual), N.ptr(w), N.ptr(b), N.ptr(running_mean),
                                                N.ptr(running_var), N.ptr(y), N.ptr(ss[:C]), N.ptr(ss[C:]), N.c_int64(R), C,
                                                N.c_float(eps), int(relu), N.stream_ptr())
            N.check(rc, "ax_batchnorm_fwd_eval")
            return y
    # torch path (CPU, other dtypes/layouts, differentiable inference)
    if training and running_mean is not None:
        with torch.no_grad():
            dims = [0] + list(range(2, x.dim()))
            xf = x.detach().float()
            running_mean.mul_(1 - momentum).add_(xf.mean(dims), alpha=momentum)
            running_var.mul_(1 - momentum).add_(xf.var(dims, unbiased=False), alpha=momentum)
        y = F.batch_norm(x, None, None, weight, bias, True, 0.0, eps)
    else:
        y = F.batch_norm(x, running_mean, running_var, weight, bias, training, 0.0, eps)
    if residual is not None:
        y = y + residual
    return torch.relu(y) if relu else y


class _MaxPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, s, p):
        n, c, h, w = x.shape
        ho, wo = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        y = torch.empty((n, c, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        need = ctx.needs_input_grad[0]
        idx = torch.empty(n * ho * wo * c, dtype=torch.uint8, device=x.device) if need else None
        rc = N.cuda().ax_maxpool2d_fwd(N.ptr(x), N.ptr(y), N.ptr(idx), n, h, w, c, k, s, p, N.stream_ptr())
        N.check(rc, "ax_maxpool2d_fwd")
        ctx.save_for_backward(idx)
        ctx.geom = (n, c, h, w, k, s, p)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        n, c, h, w, k, s, p = ctx.geom
        if not dy.is_contiguous(memory_format=torch.channels_last):
            dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty((n, c, h, w), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        rc = N.cuda().ax_maxpool2d_bwd(N.ptr(dy), N.ptr(idx), N.ptr(dx), n, h, w, c, k, s, p, N.stream_ptr())
        N.check(rc, "ax_maxpool2d_bwd")
        return dx, None, None, None


def max_pool2d(x, kernel_size: int, stride: int, padding: int):
    if (supported(x) or (x.is_cuda and N.have_gpu() and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[1] % 8 == 0
                         and x.is_contiguous(memory_format=torch.channels_last))) and kernel_size * kernel_size <= 255:
        return _MaxPool.apply(x, int(kernel_size), int(stride), int(padding))
    return F.max_pool2d(x, kernel_size, stride, padding)
