"""bf16 GEMM on the hand-written tcgen05/TMEM kernel (``csrc/kernels/gemm_tcgen05.cu``).

``gemm_bf16`` is the raw entry; ``linear`` is the autograd-aware fused Linear(+bias+activation)
that the nn layers call.  Parity: the reference's FusedLinear
(crates/axonml-fusion/src/linear.rs:111-174) and Linear forward
(crates/axonml-nn/src/layers/linear.rs:104-140).
"""
from __future__ import annotations

import torch

from .. import _native as N

ACT = {"none": 0, None: 0, "relu": 1, "gelu": 2, "sigmoid": 3, "tanh": 4, "silu": 5}


def gemm_supported(*tensors) -> bool:
    """True when the tcgen05 kernel can take these operands (bf16, CUDA sm_100, 16-byte rows)."""
    if not N.is_blackwell():
        return False
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16:
            return False
    return True


def set_pair_mode(mode: int) -> None:
    """Tile policy of the GEMM: -1 chooses per shape (default), 0 always one CTA per tile, 1 CTA
    pairs (``tcgen05 cta_group::2``, 256-row tiles) wherever the shape allows them."""
    N.cuda().ax_gemm_set_pair_mode(int(mode))


def pair_capacity() -> int:
    """CTA pairs (clusters of two) the current GPU runs at once; at most half its SM count."""
    return int(N.cuda().ax_gemm_pair_capacity())


def _as2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("expected a 2-D tensor")
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
        if t.stride(0) % 8 != 0:
            raise ValueError("row stride must be a multiple of 8 elements")
    return t


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = True,
              bias: torch.Tensor | None = None, act: str | None = None, want_aux: bool = False,
              out: torch.Tensor | None = None, bn: int = 0, max_ctas: int = 0):
    """``C = act(op(a) @ op(b) + bias)`` in bf16 with fp32 accumulation.

    ``trans_a=False``: ``a`` is ``[M,K]``; ``True``: ``a`` is ``[K,M]``.
    ``trans_b=True``:  ``b`` is ``[N,K]`` (Linear weight layout); ``False``: ``b`` is ``[K,N]``.
    With ``want_aux`` the pre-activation is returned as a second tensor.
    """
    a = _as2d(a)
    b = _as2d(b)
    if trans_a:
        K, M = a.shape
    else:
        M, K = a.shape
    if trans_b:
        Nn, Kb = b.shape
    else:
        Kb, Nn = b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if Nn % 8 != 0:
        raise ValueError("N must be a multiple of 8 for the bf16 TMA store")
    if out is None:
        out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a.device)
    aux = torch.empty_like(out) if want_aux else None
    bias_kind = 0
    if bias is not None:
        bias = bias.contiguous()
        bias_kind = 1 if bias.dtype == torch.float32 else 2
        if bias.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("bias must be fp32 or bf16")
    rc = N.cuda().ax_gemm_bf16(
        N.ptr(a), N.ptr(b), N.ptr(out), N.ptr(aux), N.ptr(bias), bias_kind, ACT[act],
        M, Nn, K, a.stride(0), b.stride(0), out.stride(0), int(trans_a), int(not trans_b),
        bn, max_ctas, N.ptr(N.status_word(a.device)), N.stream_ptr())
    N.check(rc, "ax_gemm_bf16")
    return (out, aux) if want_aux else out


def sgemm_f32(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a @ b`` in fp32 on the CUDA cores (fp32 multiply-add, fp32 accumulation): ``a`` is
    ``[M, K]`` or ``[B, M, K]``, ``b`` is ``[K, N]`` or ``[B, K, N]`` (a 2-D operand is shared by the
    whole batch).  The full-precision counterpart of the reference's cuBLAS ``sgemm`` /
    ``sgemmStridedBatched`` calls (crates/axonml-core/src/backends/cuda.rs:413-501)."""
    import ctypes
    if a.dtype != torch.float32 or b.dtype != torch.float32 or not a.is_cuda:
        raise ValueError("sgemm_f32 takes fp32 CUDA tensors")
    batch = max(a.shape[0] if a.dim() == 3 else 1, b.shape[0] if b.dim() == 3 else 1)
    a, b = a.contiguous(), b.contiguous()
    M, K = a.shape[-2:]
    Kb, Nn = b.shape[-2:]
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    shape = (batch, M, Nn) if (a.dim() == 3 or b.dim() == 3) else (M, Nn)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=a.device)
    rc = N.cuda().ax_sgemm_f32(N.ptr(a), N.ptr(b), N.ptr(out), M, Nn, K, K, Nn, Nn, batch,
                               ctypes.c_long(M * K if a.dim() == 3 else 0), ctypes.c_long(K * Nn if b.dim() == 3 else 0),
                               ctypes.c_long(M * Nn), N.stream_ptr())
    N.check(rc, "ax_sgemm_f32")
    return out
