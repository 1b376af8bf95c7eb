"""Autograd-aware fused Linear (+bias +activation) on the tcgen05 GEMM.

Forward:   y   = act(x W^T + b)              one kernel (bias/activation in the epilogue)
Backward:  dz  = dy * act'(z)                one elementwise kernel (skipped for act = none)
           dx  = dz W                        GEMM with an MN-major B operand (no transpose copy)
           dW  = dz^T x                      GEMM with MN-major A and B operands
           db  = column sums of dz           one reduction kernel

On a non-Blackwell device or a dtype other than bf16 the same maths runs through torch ops,
which is what the CPU tests and the CPU configuration use.

Parity: FusedLinear crates/axonml-fusion/src/linear.rs:20-175; Linear
crates/axonml-nn/src/layers/linear.rs:104-140.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N
from . import elementwise as E
from .gemm import gemm_bf16, gemm_supported

_ACT_FWD = {
    "none": lambda z: z,
    "relu": torch.relu,
    "gelu": lambda z: F.gelu(z, approximate="tanh"),
    "sigmoid": torch.sigmoid,
    "tanh": torch.tanh,
    "silu": F.silu,
}


def _use_kernel(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (gemm_supported(x, w) and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act, sink=None):
        ctx.sink = sink
        x2 = x.reshape(-1, x.shape[-1])
        need_z = act != "none" and (x.requires_grad or w.requires_grad)
        y = None
        gate = getattr(w, "_axon_gate", None)
        if gate is not None and gate.pending:
            # first use of a sharded unit's parameters in this pass: gather them inside this GEMM
            if gate.usable(x2, w, need_z):
                y, z = gate.gemm(x2.contiguous(), w, b, act), None
            else:
                gate.fallback()
        if y is None:
            if need_z:
                y, z = gemm_bf16(x2, w, bias=b, act=act, want_aux=True)
            else:
                y, z = gemm_bf16(x2, w, bias=b, act=act), None
        ctx.act = act
        ctx.has_bias = b is not None
        ctx.bias_dtype = b.dtype if b is not None else None
        ctx.save_for_backward(x2, w, z if z is not None else y)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, z = ctx.saved_tensors          # with activation checkpointing this recomputes the unit's forward
        gate = getattr(w, "_axon_gate", None)
        if gate is not None and gate.pending:
            gate.fallback()                   # a sharded unit whose gather is still owed (no recomputation ran)
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act != "none":
            dz = E.act_backward(dy2, z, ctx.act)
        else:
            dz = dy2
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm_bf16(dz, w, trans_b=False).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            sink = ctx.sink
            if sink is not None and sink.target().dtype == torch.bfloat16:
                # write the weight gradient straight into the sharded engine's flat buffer
                if sink.first_write():
                    gemm_bf16(dz, x2, trans_a=True, trans_b=False, out=sink.target())
                else:
                    sink.target().add_(gemm_bf16(dz, x2, trans_a=True, trans_b=False))
                sink.done()
            else:
                dw = gemm_bf16(dz, x2, trans_a=True, trans_b=False)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = E.colsum(dz).to(ctx.bias_dtype)
        return dx, dw, db, None, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           act: str = "none") -> torch.Tensor:
    """``act(x @ weight.T + bias)`` for ``weight[out, in]``; any number of leading dims."""
    act = act or "none"
    gate = getattr(weight, "_axon_gate", None)
    if gate is not None and gate.pending and not _use_kernel(x, weight):
        gate.fallback()            # a sharded unit's gather is still owed and this call cannot carry it
    if _use_kernel(x, weight):
        if bias is not None and bias.dtype not in (torch.float32, torch.bfloat16):
            bias = bias.float()
        return _LinearFn.apply(x, weight, bias, act, getattr(weight, "_axon_grad_sink", None))
    if x.is_cuda and N.is_blackwell() and torch.is_autocast_enabled():
        # autocast region with fp32 parameters: cast once, then take the kernel path
        dt = torch.get_autocast_dtype("cuda")
        if dt == torch.bfloat16 and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
            return _LinearFn.apply(x.to(dt), weight.to(dt), bias, act)
    return _ACT_FWD[act](F.linear(x, weight, bias))
