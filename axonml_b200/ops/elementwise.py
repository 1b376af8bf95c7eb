"""Python entry points of the elementwise / activation kernel set
(``csrc/kernels/elementwise.cu``).  Each function runs the hand-written kernel for CUDA fp32 /
bf16 tensors and the equivalent torch expression elsewhere (CPU, other dtypes)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N

UNARY = {"neg": 0, "abs": 1, "sqrt": 2, "exp": 3, "log": 4, "relu": 5, "sigmoid": 6, "tanh": 7,
         "gelu": 8, "silu": 9, "elu": 10, "leaky_relu": 11, "scale": 12, "add_scalar": 13,
         "pow_scalar": 14, "clamp": 15, "square": 16, "rsqrt": 17, "copy": 18}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4, "max": 5, "min": 6, "relu_bwd": 7,
          "sigmoid_bwd": 8, "tanh_bwd": 9, "gelu_bwd": 10, "silu_bwd": 11, "elu_bwd": 12,
          "leaky_relu_bwd": 13, "axpy": 14}

_UNARY_REF = {
    "neg": lambda x, a, b: -x, "abs": lambda x, a, b: x.abs(), "sqrt": lambda x, a, b: x.sqrt(),
    "exp": lambda x, a, b: x.exp(), "log": lambda x, a, b: x.log(),
    "relu": lambda x, a, b: x.relu(), "sigmoid": lambda x, a, b: x.sigmoid(),
    "tanh": lambda x, a, b: x.tanh(), "gelu": lambda x, a, b: F.gelu(x, approximate="tanh"),
    "silu": lambda x, a, b: F.silu(x), "elu": lambda x, a, b: F.elu(x, a),
    "leaky_relu": lambda x, a, b: F.leaky_relu(x, a), "scale": lambda x, a, b: x * a,
    "add_scalar": lambda x, a, b: x + a, "pow_scalar": lambda x, a, b: x.pow(a),
    "clamp": lambda x, a, b: x.clamp(a, b), "square": lambda x, a, b: x * x,
    "rsqrt": lambda x, a, b: x.rsqrt(), "copy": lambda x, a, b: x.clone(),
}


def _dt(t: torch.Tensor) -> int:
    return 1 if t.dtype == torch.bfloat16 else 0


def kernel_ok(*ts) -> bool:
    return all(t.is_cuda and t.dtype in (torch.float32, torch.bfloat16) for t in ts) and N.have_gpu()


def unary(x: torch.Tensor, op: str, p0: float = 0.0, p1: float = 0.0, out=None) -> torch.Tensor:
    if not kernel_ok(x):
        return _UNARY_REF[op](x, p0, p1)
    x = x.contiguous()
    y = torch.empty_like(x) if out is None else out
    N.check(N.cuda().ax_unary(_dt(x), UNARY[op], N.ptr(x), N.ptr(y), N.c_int64(x.numel()),
                              N.c_float(p0), N.c_float(p1), N.stream_ptr()), "ax_unary")
    return y


def _binary_ref(a, b, op, p0):
    if op == "add": return a + b
    if op == "sub": return a - b
    if op == "mul": return a * b
    if op == "div": return a / b
    if op == "pow": return a.pow(b)
    if op == "max": return torch.maximum(a, b)
    if op == "min": return torch.minimum(a, b)
    if op == "axpy": return a + p0 * b
    if op == "relu_bwd": return a * (b > 0)
    if op == "sigmoid_bwd": return a * b * (1 - b)
    if op == "tanh_bwd": return a * (1 - b * b)
    if op == "leaky_relu_bwd": return torch.where(b > 0, a, a * p0)
    if op == "elu_bwd": return torch.where(b > 0, a, a * p0 * b.exp())
    if op in ("gelu_bwd", "silu_bwd"):
        bb = b.detach().float().requires_grad_(True)
        with torch.enable_grad():
            f = F.gelu(bb, approximate="tanh") if op == "gelu_bwd" else F.silu(bb)
            (g,) = torch.autograd.grad(f, bb, a.float())
        return g.to(a.dtype)
    raise KeyError(op)


def binary(a: torch.Tensor, b: torch.Tensor, op: str, p0: float = 0.0, out=None) -> torch.Tensor:
    if not kernel_ok(a, b) or a.shape != b.shape or a.dtype != b.dtype:
        return _binary_ref(a, b, op, p0)
    a = a.contiguous()
    b = b.contiguous()
    y = torch.empty_like(a) if out is None else out
    N.check(N.cuda().ax_binary(_dt(a), BINARY[op], N.ptr(a), N.ptr(b), N.ptr(y),
                               N.c_int64(a.numel()), N.c_float(p0), N.stream_ptr()), "ax_binary")
    return y


def act_backward(dy: torch.Tensor, saved: torch.Tensor, act: str, p0: float = 0.0) -> torch.Tensor:
    """dy * act'(.) where ``saved`` is the pre-activation (relu, gelu, silu, elu, leaky_relu) or
    the activation output (sigmoid, tanh)."""
    if act in ("none", None):
        return dy
    return binary(dy, saved, act + "_bwd", p0)


def colsum(x: torch.Tensor) -> torch.Tensor:
    """fp32 column sums of a 2-D tensor (bias gradient)."""
    if not kernel_ok(x):
        return x.float().sum(0)
    if x.stride(1) != 1:
        x = x.contiguous()
    out = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
    N.check(N.cuda().ax_colsum(_dt(x), N.ptr(x), N.ptr(out), N.c_int64(x.shape[0]), x.shape[1],
                               N.c_int64(x.stride(0)), N.stream_ptr()), "ax_colsum")
    return out


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        H = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * H)
        out = torch.empty((g2.shape[0], H), dtype=gu.dtype, device=gu.device)
        N.check(N.cuda().ax_swiglu_fwd(_dt(gu), N.ptr(g2), N.ptr(out), N.c_int64(g2.shape[0]), H,
                                       N.stream_ptr()), "ax_swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], H)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        H = g2.shape[1] // 2
        d2 = dout.reshape(-1, H).contiguous()
        dgu = torch.empty_like(g2)
        N.check(N.cuda().ax_swiglu_bwd(_dt(g2), N.ptr(d2), N.ptr(g2), N.ptr(dgu),
                                       N.c_int64(g2.shape[0]), H, N.stream_ptr()), "ax_swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for a fused ``[..., 2H]`` tensor laid out gate|up."""
    H = gate_up.shape[-1] // 2
    vec = 8 if gate_up.dtype == torch.bfloat16 else 4
    if kernel_ok(gate_up) and H % vec == 0 and gate_up.is_contiguous():
        return _SwiGLU.apply(gate_up)
    g, u = gate_up.split(H, dim=-1)
    return F.silu(g) * u


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        x = x.contiguous()
        y = torch.empty_like(x)
        mask = torch.empty(x.numel(), dtype=torch.uint8, device=x.device)
        N.check(N.cuda().ax_dropout_fwd(_dt(x), N.ptr(x), N.ptr(y), N.ptr(mask),
                                        N.c_int64(x.numel()), N.c_float(p),
                                        N.ctypes.c_uint64(seed), N.ctypes.c_uint64(offset),
                                        N.stream_ptr()), "ax_dropout_fwd")
        ctx.save_for_backward(mask)
        ctx.p = p
        return y

    @staticmethod
    def backward(ctx, dy):
        (mask,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(dy)
        N.check(N.cuda().ax_dropout_bwd(_dt(dy), N.ptr(dy), N.ptr(mask), N.ptr(dx),
                                        N.c_int64(dy.numel()), N.c_float(ctx.p), N.stream_ptr()),
                "ax_dropout_bwd")
        return dx, None, None, None


_DROPOUT_CALLS = [0]


def dropout(x: torch.Tensor, p: float, training: bool = True) -> torch.Tensor:
    """Inverted dropout with a Philox counter RNG seeded from torch's generator."""
    if not training or p <= 0.0:
        return x
    if p >= 1.0:
        return torch.zeros_like(x)
    if kernel_ok(x):
        seed = int(torch.initial_seed()) & 0xFFFFFFFFFFFFFFFF
        _DROPOUT_CALLS[0] += 1
        return _Dropout.apply(x, float(p), seed, _DROPOUT_CALLS[0] << 32)
    return F.dropout(x, p, True)
