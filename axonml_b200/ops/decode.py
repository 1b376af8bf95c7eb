"""Decode-step producers of int8 activations (``csrc/kernels/decode_fused.cu``) and the
matrix-vector products that consume them (``csrc/kernels/qgemv.cu``).

A decode step at batches of up to four rows is a chain of launches of a few microseconds; these
wrappers remove the launches that only reshape data: norm, SwiGLU and the attention merge write
the int8 blocks the next matrix-vector kernel reads (no quantiser launch in between), and RoPE,
the copy of q and the KV-cache write are one launch.

Parity: the reference decodes through dequantise + fp32 matmul on the CPU
(crates/axonml-quant/src/dequantize.rs:20-125, crates/axonml-llm/src/attention.rs:19-86)."""
from __future__ import annotations

import dataclasses
import math

import torch

from .. import _native as N


@dataclasses.dataclass
class QAct:
    """Activations ``[B, K]`` quantised in blocks of 32: int8 values, block scales ``dx`` and scaled
    block sums ``sx`` (what ``ax_q4k_gemv`` / ``ax_q80_gemv`` read)."""
    x8: torch.Tensor
    dx: torch.Tensor
    sx: torch.Tensor
    B: int
    K: int

    @staticmethod
    def empty(B: int, K: int, device) -> "QAct":
        return QAct(torch.empty(B * K, dtype=torch.int8, device=device),
                    torch.empty(B * (K // 32), dtype=torch.float32, device=device),
                    torch.empty(B * (K // 32), dtype=torch.float32, device=device), B, K)

    def dequantize(self) -> torch.Tensor:
        """fp32 ``[B, K]`` (for tests)."""
        return (self.x8.view(self.B, self.K // 32, 32).float() * self.dx.view(self.B, -1, 1)).view(self.B, self.K)


def supported(x: torch.Tensor) -> bool:
    return N.is_blackwell() and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 32 == 0


def quantize_rows(x: torch.Tensor) -> QAct:
    B, K = x.shape
    if x.stride(1) != 1 or x.stride(0) % 8:
        x = x.contiguous()
    q = QAct.empty(B, K, x.device)
    N.check(N.cuda().ax_q8_rows(N.ptr(x), N.c_int64(x.stride(0)), N.ptr(q.x8), N.ptr(q.dx), N.ptr(q.sx), B, K,
                                N.stream_ptr()), "ax_q8_rows")
    return q


def rms_norm_q8(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                want_bf16: bool = False):
    """``q8(rmsnorm(x + residual) * weight)``.  Returns ``(QAct, stream, h)``: ``stream`` is the
    updated residual stream ``x + residual`` (``x`` itself without a residual), ``h`` the bf16
    normalised rows when ``want_bf16``."""
    B, K = x.shape
    assert x.is_contiguous() and (residual is None or residual.is_contiguous())
    w_kind = 1 if weight.dtype == torch.float32 else 2
    if weight.dtype not in (torch.float32, torch.bfloat16):
        weight, w_kind = weight.float(), 1
    q = QAct.empty(B, K, x.device)
    stream = torch.empty_like(x) if residual is not None else x
    h = torch.empty_like(x) if want_bf16 else None
    N.check(N.cuda().ax_rmsnorm_q8(N.ptr(x), N.c_int64(K), N.ptr(residual), N.c_int64(K), N.ptr(weight), w_kind,
                                   N.c_float(eps), N.ptr(stream if residual is not None else None), N.c_int64(K),
                                   N.ptr(h), N.c_int64(K), N.ptr(q.x8), N.ptr(q.dx), N.ptr(q.sx), B, K, N.stream_ptr()),
            "ax_rmsnorm_q8")
    return q, stream, h


def swiglu_q8(gate_up: torch.Tensor) -> QAct:
    B, F2 = gate_up.shape
    F = F2 // 2
    assert gate_up.is_contiguous()
    q = QAct.empty(B, F, gate_up.device)
    N.check(N.cuda().ax_swiglu_q8(N.ptr(gate_up), N.c_int64(F2), N.ptr(q.x8), N.ptr(q.dx), N.ptr(q.sx), B, F,
                                  N.stream_ptr()), "ax_swiglu_q8")
    return q


def rope_kv_write(qkv: torch.Tensor, cos, sin, positions, k_cache, v_cache, block_table, seq_ids, Hq: int, Hkv: int,
                  page_size: int) -> torch.Tensor:
    """``qkv`` [B, Hq + 2 Hkv, 128] bf16: rotates the q and k heads at ``positions``, returns the
    rotated q ``[B, Hq, 128]`` and writes the rotated k and the v of every token into the pages of
    its sequence."""
    B = qkv.shape[0]
    assert qkv.stride(2) == 1 and qkv.stride(1) == 128
    q = torch.empty((B, Hq, 128), dtype=torch.bfloat16, device=qkv.device)
    N.check(N.cuda().ax_rope_kv_write(N.ptr(qkv), N.c_int64(qkv.stride(0)), N.ptr(cos), N.ptr(sin), N.ptr(positions),
                                      N.ptr(q), N.ptr(k_cache), N.ptr(v_cache), N.ptr(block_table), N.ptr(seq_ids), B, Hq,
                                      Hkv, 128, page_size, block_table.shape[1], N.stream_ptr()), "ax_rope_kv_write")
    return q


def gemv_ok(qweight, B: int) -> bool:
    """Whether ``qgemv`` has a kernel for this weight at this batch."""
    from ..quant.types import QuantType
    Nn, K = qweight.shape
    if not qweight.data.is_cuda or K % 256:
        return False
    if qweight.quant_type is QuantType.Q4_K and qweight.layout in ("ggml", "tile128"):
        return B <= 4
    return (qweight.quant_type is QuantType.Q8_0 and qweight.layout == "tile128" and Nn >= 128 * 148 and B <= 4)


def qgemv(a: QAct, qweight, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``a`` times the quantised ``W[N, K]``^T -> ``[B, N]``, the activations already int8."""
    from ..quant.types import QuantType
    Nn, K = qweight.shape
    assert K == a.K
    out = torch.empty((a.B, Nn), dtype=out_dtype, device=a.x8.device)
    if qweight.quant_type is QuantType.Q4_K:
        rc = N.cuda().ax_q4k_gemv(N.ptr(qweight.data), int(qweight.layout == "tile128"), N.ptr(None), N.c_int64(0), N.ptr(a.x8),
                                  N.ptr(a.dx), N.ptr(a.sx), N.ptr(out), int(out_dtype == torch.bfloat16), a.B, Nn, K,
                                  N.stream_ptr())
        N.check(rc, "ax_q4k_gemv")
    else:
        rc = N.cuda().ax_q80_gemv(N.ptr(qweight.data), N.ptr(None), N.c_int64(0), N.ptr(a.x8), N.ptr(a.dx), N.ptr(a.sx),
                                  N.ptr(out), int(out_dtype == torch.bfloat16), a.B, Nn, K,
                                  N.ptr(N.status_word(out.device)), N.stream_ptr())
        N.check(rc, "ax_q80_gemv")
    return out


def decode_attention_q8(q, k_cache, v_cache, block_table, ctx_lens, page_size: int, scale: float | None = None):
    """Paged decode attention whose merge kernel also writes the int8 form of the result: returns
    ``(out [B, Hq, 128] bf16, QAct over [B, Hq * 128])``."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    capacity = block_table.shape[1] * page_size
    splits = max(2, min(296 // max(B * Hkv, 1), (capacity + 31) // 32, 64))
    ws = torch.empty(B * Hq * splits * (D + 2), dtype=torch.float32, device=q.device)
    a = QAct.empty(B, Hq * D, q.device)
    rc = N.cuda().ax_paged_decode_attention(N.ptr(q), N.ptr(k_cache), N.ptr(v_cache), N.ptr(out), N.ptr(block_table),
                                            N.ptr(ctx_lens), B, Hq, Hkv, D, page_size, block_table.shape[1],
                                            N.c_float(scale), N.c_int64(q.stride(0)), N.c_int64(out.stride(0)), splits,
                                            N.ptr(ws), k_cache.shape[0], N.ptr(N.status_word(q.device)), N.ptr(a.x8),
                                            N.ptr(a.dx), N.ptr(a.sx), N.stream_ptr())
    N.check(rc, "ax_paged_decode_attention")
    return out, a
