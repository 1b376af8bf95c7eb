"""GPU block quantisation, dequantisation and the dequantising matmul
(``csrc/kernels/quant.cu``, ``qgemm.cu``)."""
from __future__ import annotations

import os

import torch

from .. import _native as N


def quantize_cuda(x: torch.Tensor, quant_type) -> torch.Tensor:
    """fp32/bf16 CUDA tensor -> packed uint8 blocks (GGML layout), on the GPU for every block format
    of the package (Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q4_K); other inputs go through the CPU codec."""
    from ..quant.types import QuantType
    n = x.numel()
    nbytes = n // quant_type.block_size() * quant_type.bytes_per_block()
    if quant_type.codec_id() in (0, 1, 2, 3, 4, 5) and x.is_cuda and x.dtype in (torch.float32, torch.bfloat16):
        xc = x.contiguous()
        out = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        rc = N.cuda().ax_quantize_cuda(quant_type.codec_id(), int(xc.dtype == torch.bfloat16), N.ptr(xc), N.ptr(out),
                                       N.c_int64(n), N.stream_ptr())
        N.check(rc, "ax_quantize_cuda")
        return out
    from ..quant.quantize import quantize_tensor
    return quantize_tensor(x.detach().float().cpu(), quant_type).data.to(x.device)


def dequantize_cuda(data: torch.Tensor, quant_type, numel: int, dtype=torch.float32) -> torch.Tensor:
    out_dt = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    y = torch.empty(numel, dtype=out_dt, device=data.device)
    rc = N.cuda().ax_dequantize_cuda(quant_type.codec_id(), int(out_dt == torch.bfloat16), N.ptr(data), N.ptr(y),
                                     N.c_int64(numel), N.stream_ptr())
    N.check(rc, "ax_dequantize_cuda")
    return y if out_dt == dtype else y.to(dtype)


def tile_weight(qweight):
    """Repacks a row-major quantised ``[N, K]`` weight (Q4_K / Q8_0, K % 256 == 0) so that the 128
    rows of a tile are contiguous for every 256-wide k block: ``[N/128][K/256][128][bytes]``.  The
    dequantising matmul then fetches a whole stage with one bulk copy instead of 128 small ones.
    Rows are padded to a multiple of 128 with zero blocks."""
    from ..quant.types import QuantizedTensor
    Nn, K = qweight.shape
    qt = qweight.quant_type
    sb = 256 // qt.block_size() * qt.bytes_per_block()          # bytes of one row within a k block
    kb = K // 256
    d = qweight.data.view(Nn, kb, sb)
    pad = (-Nn) % 128
    if pad:
        d = torch.cat([d, torch.zeros((pad, kb, sb), dtype=torch.uint8, device=d.device)], 0)
    d = d.view(-1, 128, kb, sb).permute(0, 2, 1, 3).contiguous()
    return QuantizedTensor([Nn, K], qt, d.view(-1), "tile128")


def untile_weight(qweight):
    from ..quant.types import QuantizedTensor
    Nn, K = qweight.shape
    qt = qweight.quant_type
    sb = 256 // qt.block_size() * qt.bytes_per_block()
    kb = K // 256
    d = qweight.data.view(-1, kb, 128, sb).permute(0, 2, 1, 3).reshape(-1, kb * sb)[:Nn].contiguous()
    return QuantizedTensor([Nn, K], qt, d.view(-1), "ggml")


def qgemm_supported(x: torch.Tensor, qweight) -> bool:
    from ..quant.types import QuantType
    return (N.is_blackwell() and x.is_cuda and x.dtype == torch.bfloat16 and qweight.data.is_cuda
            and qweight.quant_type in (QuantType.Q4_K, QuantType.Q8_0) and len(qweight.shape) == 2
            and qweight.shape[1] % 256 == 0 and qweight.layout in ("ggml", "tile128"))


def qgemm(x: torch.Tensor, qweight, out: torch.Tensor | None = None, splits: int = 0,
          out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``x[B, K]`` (bf16, B <= 64 per launch) times the quantised ``W[N, K]``^T -> fp32 ``[B, N]``.
    Larger batches are processed in slices of 64 rows.  ``out_dtype=torch.bfloat16`` lets the
    matrix-vector kernels write bf16 themselves; the tensor-core kernel accumulates split-k partial
    sums in fp32 and is converted afterwards."""
    Nn, K = qweight.shape
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    B = x2.shape[0]
    from ..quant.types import QuantType
    if B <= 4 and qweight.quant_type is QuantType.Q4_K and os.environ.get("AXONML_QGEMV", "1") != "0":
        # decode-sized batches: matrix-vector kernel (dp4a on int8 activations, weights read once from HBM)
        if out is None:
            out = torch.empty((B, Nn), dtype=out_dtype, device=x.device)
        x8 = torch.empty(B * K, dtype=torch.int8, device=x.device)
        dxs = torch.empty(2 * B * (K // 32), dtype=torch.float32, device=x.device)
        rc = N.cuda().ax_q4k_gemv(N.ptr(qweight.data), int(qweight.layout == "tile128"), N.ptr(x2), N.c_int64(x2.stride(0)),
                                  N.ptr(x8), N.ptr(dxs), N.ptr(dxs[B * (K // 32):]), N.ptr(out),
                                  int(out.dtype == torch.bfloat16), B, Nn, K, N.stream_ptr())
        N.check(rc, "ax_q4k_gemv")
        return out.view(*x.shape[:-1], Nn)
    if (B <= 4 and qweight.quant_type is QuantType.Q8_0 and qweight.layout == "tile128" and Nn >= 128 * 148
            and os.environ.get("AXONML_QGEMV", "1") != "0"):
        # wide Q8_0 matrices (the LM head): one CTA per 128-row tile streams its k blocks through shared memory
        if out is None:
            out = torch.empty((B, Nn), dtype=out_dtype, device=x.device)
        x8 = torch.empty(B * K, dtype=torch.int8, device=x.device)
        dxs = torch.empty(2 * B * (K // 32), dtype=torch.float32, device=x.device)
        rc = N.cuda().ax_q80_gemv(N.ptr(qweight.data), N.ptr(x2), N.c_int64(x2.stride(0)), N.ptr(x8), N.ptr(dxs),
                                  N.ptr(dxs[B * (K // 32):]), N.ptr(out), int(out.dtype == torch.bfloat16), B, Nn, K,
                                  N.ptr(N.status_word(x.device)), N.stream_ptr())
        N.check(rc, "ax_q80_gemv")
        return out.view(*x.shape[:-1], Nn)
    if out is None:
        out = torch.zeros((B, Nn), dtype=torch.float32, device=x.device)
    for b0 in range(0, B, 64):
        xs = x2[b0:b0 + 64]
        rc = N.cuda().ax_qgemm(qweight.quant_type.codec_id(), N.ptr(qweight.data), N.ptr(xs), N.ptr(out[b0:b0 + 64]),
                               xs.shape[0], Nn, K, xs.stride(0), splits, int(qweight.layout == "tile128"),
                               N.ptr(N.status_word(x.device)), N.stream_ptr())
        N.check(rc, "ax_qgemm")
    if out.dtype != out_dtype:
        out = out.to(out_dtype)
    return out.view(*x.shape[:-1], Nn)


def qlinear(x: torch.Tensor, qweight, bias=None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """Linear layer on a quantised weight: the fused dequant-matmul for up to a few hundred rows,
    dequantise + tcgen05 GEMM beyond that (compute-bound prefill)."""
    rows = x.numel() // x.shape[-1]
    if qgemm_supported(x, qweight) and rows <= 256:
        if bias is None:
            return qgemm(x, qweight, out_dtype=out_dtype)
        return (qgemm(x, qweight) + bias.float()).to(out_dtype)
    from ..quant.quantize import dequantize_tensor
    from .linear import linear
    if qweight.layout == "tile128":
        qweight = untile_weight(qweight)
    w = dequantize_tensor(qweight, x.dtype if x.is_floating_point() else torch.float32)
    return linear(x, w, bias).to(out_dtype)
