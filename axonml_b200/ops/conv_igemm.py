"""Implicit-GEMM convolution on tcgen05 (``csrc/kernels/conv_igemm.cu``).

Forward and data gradient run without an im2col matrix: the kernel's TMA producer loads, per
filter tap, the tile's box of NHWC input pixels shifted by the tap (zero padding is the TMA
out-of-range fill).  A strided convolution reads the input through ``sh * sw`` parity views (tensor
maps over every sh-th row and sw-th column), in which the pixels of one tap are again a plain box.
The data gradient of a stride-1 convolution is the same kernel applied to the output gradient with
the filter rotated by 180 degrees and its channel dims exchanged; that of a strided one is one
launch per parity class of the input pixels, each with only the taps that reach the class and a
strided view of ``dx`` as its output, so no multiplication by an inserted zero is computed.  The
weight gradient is a second implicit GEMM whose reduction dimension is the pixels.

Layout contract: activations are bf16 in channels-last memory format (NCHW shape, NHWC storage),
weights ``[cout, cin, kh, kw]`` in any float dtype (converted to ``[cout, kh, kw, cin]`` bf16).

Parity: Conv2d forward crates/axonml-nn/src/layers/conv.rs:256-337 and the WGSL direct-conv
shader (wgpu_backend.rs:1364-1427); the reference has no convolution backward."""
from __future__ import annotations

import torch

from .. import _native as N
from .gemm import ACT


def supported(x, weight, stride, padding, dilation=(1, 1), groups: int = 1) -> bool:
    if not (N.is_blackwell() and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16):
        return False
    sh, sw = tuple(stride)
    if sh < 1 or sw < 1 or sh * sw > 4 or tuple(dilation) != (1, 1) or groups != 1:
        return False
    cout, cin, kh, kw = weight.shape
    if cin % 64 or cout % 64 or kh * kw > 64:
        return False
    if not x.is_contiguous(memory_format=torch.channels_last):
        return False
    n, _, h, w = x.shape
    if h < sh or w < sw or h + 2 * padding[0] < kh or w + 2 * padding[1] < kw:
        return False
    ho, wo = out_size(h, w, (kh, kw), stride, padding)
    return n * ho * wo >= 128


def out_size(h, w, kernel_size, stride, padding):
    return ((h + 2 * padding[0] - kernel_size[0]) // stride[0] + 1,
            (w + 2 * padding[1] - kernel_size[1]) // stride[1] + 1)


def _ohwi(weight: torch.Tensor) -> torch.Tensor:
    """[cout, cin, kh, kw] -> contiguous [cout, kh, kw, cin] bf16."""
    return weight.detach().permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()


def fprop(x, w_ohwi, bias, padding, act: str = "none", stride=(1, 1)):
    """x: NCHW-shaped channels-last bf16; w_ohwi: [cout, kh, kw, cin] bf16.  Returns the
    channels-last result."""
    n, cin, h, w = x.shape
    cout, kh, kw, _ = w_ohwi.shape
    ho, wo = out_size(h, w, (kh, kw), stride, padding)
    y = torch.empty((n, cout, ho, wo), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
    bias_kind = 0
    if bias is not None:
        bias = bias.detach().contiguous()
        bias_kind = 1 if bias.dtype == torch.float32 else 2
        if bias.dtype not in (torch.float32, torch.bfloat16):
            bias, bias_kind = bias.float(), 1
    rc = N.cuda().ax_conv2d_fprop(N.ptr(x), N.ptr(w_ohwi), N.ptr(y), N.ptr(bias), bias_kind, ACT[act], n, h, w, cin,
                                  cout, kh, kw, padding[0], padding[1], stride[0], stride[1], 0,
                                  N.ptr(N.status_word(x.device)), N.stream_ptr())
    N.check(rc, "ax_conv2d_fprop")
    return y


def dgrad_strided(dy, weight, in_hw, stride, padding):
    """Data gradient ``[n, cin, h, w]`` (channels-last bf16) of a strided convolution.  Input pixel
    ``(sh*i + a, sw*j + b)`` only meets the filter rows ``r = a + ph (mod sh)`` and columns
    ``s = b + pw (mod sw)``; each of the ``sh * sw`` classes is a stride-1 problem over ``dy`` with
    that subset of taps."""
    n, cout, ho, wo = dy.shape
    _, cin, kh, kw = weight.shape
    h, w = in_hw
    sh, sw = stride
    ph, pw = padding
    # the filter rows that reach class a are r0, r0 + sh, ... with r0 = (a + ph) mod sh: a strided slice
    classes = []
    for a in range(sh):
        for b in range(sw):
            classes.append((a, b, range((a + ph) % sh, kh, sh), range((b + pw) % sw, kw, sw)))
    every_pixel_written = all(len(rr) and len(cc) for _, _, rr, cc in classes)
    dx = torch.empty((n, cin, h, w), dtype=torch.bfloat16, device=dy.device, memory_format=torch.channels_last)
    if not every_pixel_written:
        dx.zero_()
    wb = weight.detach().to(torch.bfloat16)
    import ctypes
    for a, b, rr, cc in classes:
        ntaps = len(rr) * len(cc)
        if ntaps == 0:
            continue
        wc = wb[:, :, rr.start::sh, cc.start::sw].permute(1, 2, 3, 0).contiguous()    # [cin, rows, cols, cout]
        dh = (ctypes.c_int * ntaps)(*[(a + ph - r) // sh for r in rr for _ in cc])
        dw = (ctypes.c_int * ntaps)(*[(b + pw - s) // sw for _ in rr for s in cc])
        rc = N.cuda().ax_conv2d_dgrad_class(N.ptr(dy), N.ptr(wc), N.ptr(dx), n, h, w, cin, ho, wo, cout, sh, sw, a, b,
                                            ntaps, dh, dw, 0, N.ptr(N.status_word(dy.device)), N.stream_ptr())
        N.check(rc, "ax_conv2d_dgrad_class")
    return dx


def wgrad(dy, x, kernel_size, padding, stride=(1, 1)):
    """Weight gradient ``[cout, cin, kh, kw]`` (fp32) from the channels-last bf16 output gradient and
    input: pixels are the reduction dim of an implicit GEMM, split over CTAs with fp32 global
    reductions."""
    n, cin, h, w = x.shape
    cout = dy.shape[1]
    kh, kw = kernel_size
    dw = torch.zeros((cout, kh, kw, cin), dtype=torch.float32, device=x.device)
    rc = N.cuda().ax_conv2d_wgrad(N.ptr(dy), N.ptr(x), N.ptr(dw), n, h, w, cin, cout, kh, kw, padding[0], padding[1],
                                  stride[0], stride[1], 0, N.ptr(N.status_word(x.device)), N.stream_ptr())
    N.check(rc, "ax_conv2d_wgrad")
    return dw.permute(0, 3, 1, 2).contiguous()


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, padding, stride=(1, 1)):
        ctx.padding = tuple(padding)
        ctx.stride = tuple(stride)
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return fprop(x, _ohwi(weight), bias, padding, stride=ctx.stride)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        ph, pw = ctx.padding
        cout, cin, kh, kw = weight.shape
        if not dy.is_contiguous(memory_format=torch.channels_last):
            dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if ctx.stride == (1, 1):
                # rotate the filter by 180 degrees and swap its channel roles: [cin, kh, kw, cout]
                w_t = weight.detach().flip(2, 3).permute(1, 2, 3, 0).to(torch.bfloat16).contiguous()
                dx = fprop(dy, w_t, None, (kh - 1 - ph, kw - 1 - pw))
            else:
                dx = dgrad_strided(dy, weight, x.shape[2:], ctx.stride, (ph, pw))
        if ctx.needs_input_grad[1]:
            dw = wgrad(dy, x, (kh, kw), (ph, pw), ctx.stride).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(dim=(0, 2, 3)).to(ctx.bias_dtype)
        return dx, dw, db, None, None


def conv2d(x, weight, bias, stride, padding):
    if weight.shape[1] < 64:
        return _ThinConvFn.apply(x, weight, bias, tuple(stride), tuple(padding))
    return _ConvFn.apply(x, weight, bias, tuple(padding), tuple(stride))


def conv2d_supported(x, weight, stride, padding) -> bool:
    """Whether ``conv2d`` takes this call (the nn layer falls back to the torch convolution otherwise)."""
    return supported(x, weight, stride, padding) or thin_supported(x, weight, stride, padding)


# ------------------------------------------------------------------------------ one-dimensional convolutions
def _as_2d(x):
    """``[N, C, L]`` -> ``[N, C, 1, L]`` in channels-last storage (N, L, C): a view when ``x`` already
    is the squeezed result of an earlier call, one transposing copy otherwise."""
    return x.unsqueeze(2).contiguous(memory_format=torch.channels_last)


def conv1d_supported(x, weight, stride: int, padding: int) -> bool:
    if not (x.dim() == 3 and x.is_cuda and x.dtype == torch.bfloat16 and N.is_blackwell()):
        return False
    n, c, l = x.shape
    cout, cin, k = weight.shape
    if stride < 1 or stride > 4 or cin != c or cin % 64 or cout % 64 or k > 64 or l < stride or l + 2 * padding < k:
        return False
    return n * ((l + 2 * padding - k) // stride + 1) >= 128


def conv1d(x, weight, bias, stride: int, padding: int):
    """Conv1d on the implicit-GEMM kernels: the sequence is the width of an image of height one
    (forward, data gradient and weight gradient are those of ``conv2d``).  The result is a
    ``[N, Cout, Lo]`` view of channels-last storage, so a stack of such layers never transposes."""
    y = _ConvFn.apply(_as_2d(x), weight.unsqueeze(2), bias, (0, padding), (1, stride))
    return y.squeeze(2)


# ------------------------------------------------------------------------------ thin inputs (RGB stem)
def thin_supported(x, weight, stride, padding) -> bool:
    """Convolutions with fewer than 64 input channels (any stride): patches are gathered by the
    im2col kernel and multiplied by the tcgen05 GEMM."""
    if not (N.is_blackwell() and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16):
        return False
    cout, cin, kh, kw = weight.shape
    if cin >= 64 or cout % 8 or kh * ((kw * cin + 7) // 8 * 8) > 1024 or stride[0] != stride[1]:
        return False
    if not x.is_contiguous(memory_format=torch.channels_last):
        return False
    n, _, h, w = x.shape
    ho = (h + 2 * padding[0] - kh) // stride[0] + 1
    wo = (w + 2 * padding[1] - kw) // stride[1] + 1
    return ho > 0 and wo > 0 and n * ho * wo >= 128


def _thin_patches(x, kernel_size, stride, padding):
    """The patch matrix ``[n*ho*wo, kp]`` of a thin input, with its row layout (rp, kp)."""
    n, cin, h, w = x.shape
    kh, kw = kernel_size
    ho, wo = out_size(h, w, kernel_size, stride, padding)
    rp = (kw * cin + 7) // 8 * 8                      # one filter row of a patch, padded to 16-byte chunks
    kp = (kh * rp + 63) // 64 * 64
    col = torch.empty((n * ho * wo, kp), dtype=torch.bfloat16, device=x.device)
    rc = N.cuda().ax_im2col_nhwc(N.ptr(x), N.ptr(col), n, h, w, cin, kh, kw, stride[0], padding[0], padding[1], rp, kp,
                                 N.stream_ptr())
    N.check(rc, "ax_im2col_nhwc")
    return col, rp, kp, ho, wo


def thin_wgrad(dy, x, kernel_size, stride, padding):
    """Weight gradient ``[cout, cin, kh, kw]`` (fp32) of a thin-input convolution: the patches are
    gathered again (they are 20 times the input, too large to keep from the forward) and the
    pixel-reduction kernel multiplies them with ``dy`` as a 1x1 problem over ``kp`` channels."""
    n, cin, h, w = x.shape
    kh, kw = kernel_size
    cout = dy.shape[1]
    col, rp, kp, ho, wo = _thin_patches(x, kernel_size, stride, padding)
    dw = torch.zeros((cout, kp), dtype=torch.float32, device=x.device)
    rc = N.cuda().ax_conv2d_wgrad(N.ptr(dy), N.ptr(col), N.ptr(dw), n, ho, wo, kp, cout, 1, 1, 0, 0, 1, 1, 0,
                                  N.ptr(N.status_word(x.device)), N.stream_ptr())
    N.check(rc, "ax_conv2d_wgrad")
    dw = dw[:, :kh * rp].reshape(cout, kh, rp)[:, :, :kw * cin].reshape(cout, kh, kw, cin)
    return dw.permute(0, 3, 1, 2).contiguous()


def thin_fprop(x, weight, bias, stride, padding):
    from .gemm import gemm_bf16
    n, cin, h, w = x.shape
    cout, _, kh, kw = weight.shape
    col, rp, kp, ho, wo = _thin_patches(x, (kh, kw), stride, padding)
    w_rows = torch.zeros((cout, kh, rp), dtype=torch.bfloat16, device=x.device)
    w_rows[:, :, :kw * cin] = weight.detach().permute(0, 2, 3, 1).reshape(cout, kh, kw * cin)   # (kh | kw, cin) as the patches
    w2d = torch.zeros((cout, kp), dtype=torch.bfloat16, device=x.device)
    w2d[:, :kh * rp] = w_rows.reshape(cout, kh * rp)
    y = torch.empty((n, cout, ho, wo), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
    out2d = y.permute(0, 2, 3, 1).reshape(n * ho * wo, cout)                      # a view: NHWC storage
    if bias is not None and bias.dtype not in (torch.float32, torch.bfloat16):
        bias = bias.float()
    gemm_bf16(col, w2d, bias=None if bias is None else bias.detach(), out=out2d)
    return y


class _ThinConvFn(torch.autograd.Function):
    """Forward and weight gradient on this package's kernels.  A data gradient (rarely wanted: the
    layer usually reads the network input) comes from the library convolution backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding):
        ctx.stride, ctx.padding = stride, padding
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return thin_fprop(x, weight, bias, stride, padding)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        if not dy.is_contiguous(memory_format=torch.channels_last):
            dy = dy.contiguous(memory_format=torch.channels_last)
        cout, _, kh, kw = weight.shape
        dx = dw = None
        native_dw = ctx.needs_input_grad[1] and cout % 64 == 0
        if native_dw:
            dw = thin_wgrad(dy, x, (kh, kw), ctx.stride, ctx.padding)
        mask = (ctx.needs_input_grad[0], ctx.needs_input_grad[1] and not native_dw, False)
        if mask[0] or mask[1]:
            dx, dw_lib, _ = torch.ops.aten.convolution_backward(dy, x, weight.detach().to(torch.bfloat16), None,
                                                                list(ctx.stride), list(ctx.padding), [1, 1], False,
                                                                [0, 0], 1, list(mask))
            dw = dw if native_dw else dw_lib
        db = dy.float().sum(dim=(0, 2, 3)).to(ctx.bias_dtype) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, (dw.to(weight.dtype) if dw is not None else None), db, None, None
