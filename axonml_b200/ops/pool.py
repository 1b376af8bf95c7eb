"""Average pooling on the hand-written kernels (``csrc/kernels/avgpool.cu``), with the window rules
of the reference (crates/axonml-nn/src/layers/pooling.rs:296-445): ``avg_pool2d`` divides by the
number of pixels inside the image unless ``count_include_pad`` is set; ``adaptive_avg_pool2d`` uses
windows ``[floor(o*H/OH), floor((o+1)*H/OH))``, which partition the image.  CUDA tensors (fp32 or
bf16, NCHW or channels-last) run the kernels forward and backward; other tensors evaluate the same
rules with torch ops.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from .. import _native as N


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _kernel_ok(x) -> bool:
    return x.is_cuda and x.dim() == 4 and x.dtype in (torch.float32, torch.bfloat16) and N.have_gpu()


def _layout(x):
    """(dense tensor, channels_last flag) without a copy when x is dense in either layout."""
    if x.is_contiguous():
        return x, 0
    if x.is_contiguous(memory_format=torch.channels_last):
        return x, 1
    return x.contiguous(), 0


def _launch(backward, src, dst, dims, win, adaptive, count_pad, cl):
    rc = N.cuda().ax_avgpool2d(int(backward), 1 if src.dtype == torch.bfloat16 else 0, N.ptr(src), N.ptr(dst),
                               (ctypes.c_int * 6)(*dims), (ctypes.c_int * 6)(*win), int(adaptive), int(count_pad),
                               int(cl), N.stream_ptr())
    N.check(rc, "ax_avgpool2d")


class _AvgPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_hw, win, adaptive, count_pad):
        x, cl = _layout(x)
        n, c, h, w = x.shape
        oh, ow = out_hw
        fmt = torch.channels_last if cl else torch.contiguous_format
        y = torch.empty((n, c, oh, ow), dtype=x.dtype, device=x.device, memory_format=fmt)
        ctx.args = ((n, c, h, w, oh, ow), win, adaptive, count_pad, cl)
        _launch(False, x, y, (n, c, h, w, oh, ow), win, adaptive, count_pad, cl)
        return y

    @staticmethod
    def backward(ctx, dy):
        dims, win, adaptive, count_pad, cl = ctx.args
        fmt = torch.channels_last if cl else torch.contiguous_format
        dy = dy.contiguous(memory_format=fmt)
        dx = torch.empty(dims[:4], dtype=dy.dtype, device=dy.device, memory_format=fmt)
        _launch(True, dy, dx, dims, win, adaptive, count_pad, cl)
        return dx, None, None, None, None


def avg_pool2d(x, kernel_size, stride=None, padding=0, count_include_pad: bool = False):
    kh, kw = _pair(kernel_size)
    sh, sw = _pair(kernel_size if stride is None else stride)
    ph, pw = _pair(padding)
    if _kernel_ok(x):
        h, w = x.shape[2:]
        oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
        return _AvgPool.apply(x, (oh, ow), (kh, kw, sh, sw, ph, pw), False, count_include_pad)
    return F.avg_pool2d(x, (kh, kw), (sh, sw), (ph, pw), count_include_pad=count_include_pad)


def avg_pool1d(x, kernel_size: int, stride=None, padding: int = 0, count_include_pad: bool = False):
    """[N, C, L] -> [N, C, OL]: the 2-D kernel with a height of one."""
    s = kernel_size if stride is None else stride
    if x.is_cuda and x.dim() == 3 and x.dtype in (torch.float32, torch.bfloat16) and N.have_gpu():
        return avg_pool2d(x.unsqueeze(2), (1, kernel_size), (1, s), (0, padding), count_include_pad).squeeze(2)
    return F.avg_pool1d(x, kernel_size, s, padding, count_include_pad=count_include_pad)


def _axis_matrix(size: int, out: int, device, dtype):
    """[out, size] averaging matrix of the window rule [floor(o*size/out), floor((o+1)*size/out))."""
    m = torch.zeros(out, size, device=device, dtype=dtype)
    for o in range(out):
        lo, hi = (o * size) // out, ((o + 1) * size) // out
        if hi > lo:
            m[o, lo:hi] = 1.0 / (hi - lo)
    return m


def adaptive_avg_pool2d(x, output_size):
    oh, ow = _pair(output_size)
    if _kernel_ok(x):
        return _AvgPool.apply(x, (oh, ow), (1, 1, 1, 1, 0, 0), True, False)
    h, w = x.shape[-2:]
    cd = x.dtype if x.dtype in (torch.float32, torch.float64) else torch.float32
    ah, aw = _axis_matrix(h, oh, x.device, cd), _axis_matrix(w, ow, x.device, cd)
    return torch.einsum("oh,...hw,pw->...op", ah, x.to(cd), aw).to(x.dtype)
