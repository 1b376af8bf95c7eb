"""Paged KV cache kernels (``csrc/kernels/paged_attn.cu``): scatter new K/V rows into pages, decode
attention through a block table.  CPU tensors use the same maths with torch ops."""
from __future__ import annotations

import math

import torch

from .. import _native as N


def kv_write(k, v, k_cache, v_cache, block_table, seq_ids, positions, page_size: int) -> None:
    """k, v: [T, Hkv, D]; caches: [pages, page_size, Hkv, D]; block_table: [B, max_pages] int32;
    seq_ids / positions: [T] int32 (sequence and position of every token)."""
    T, Hkv, D = k.shape
    if k.is_cuda and N.have_gpu() and k.dtype == torch.bfloat16:
        if k.stride(2) != 1 or k.stride(1) != D:
            k = k.contiguous()
        if v.stride(2) != 1 or v.stride(1) != D:
            v = v.contiguous()
        rc = N.cuda().ax_paged_kv_write(N.ptr(k), N.ptr(v), N.ptr(k_cache), N.ptr(v_cache), N.ptr(block_table),
                                        N.ptr(seq_ids), N.ptr(positions), T, Hkv, D, N.c_int64(k.stride(0)),
                                        N.c_int64(v.stride(0)), page_size, block_table.shape[1], N.stream_ptr())
        N.check(rc, "ax_paged_kv_write")
        return
    pages = block_table[seq_ids.long(), (positions // page_size).long()].long()
    slots = (positions % page_size).long()
    k_cache[pages, slots] = k.to(k_cache.dtype)
    v_cache[pages, slots] = v.to(v_cache.dtype)


def decode_attention(q, k_cache, v_cache, block_table, ctx_lens, page_size: int, scale: float | None = None):
    """q: [B, Hq, D] -> [B, Hq, D]; every sequence attends to its first ``ctx_lens[b]`` cached tokens."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if q.is_cuda and N.have_gpu() and q.dtype == torch.bfloat16 and D == 128 and Hq // Hkv in (1, 2, 4, 8):
        q = q.contiguous()
        out = torch.empty_like(q)
        # context splits: enough CTAs for two per SM, at most one split per 32 tokens of capacity
        capacity = block_table.shape[1] * page_size
        splits = max(1, min(296 // max(B * Hkv, 1), (capacity + 31) // 32, 64))
        ws = torch.empty(B * Hq * splits * (D + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
        rc = N.cuda().ax_paged_decode_attention(N.ptr(q), N.ptr(k_cache), N.ptr(v_cache), N.ptr(out), N.ptr(block_table),
                                                N.ptr(ctx_lens), B, Hq, Hkv, D, page_size, block_table.shape[1],
                                                N.c_float(scale), N.c_int64(q.stride(0)), N.c_int64(out.stride(0)),
                                                splits, N.ptr(ws) if ws is not None else None, k_cache.shape[0],
                                                N.ptr(N.status_word(q.device)), N.ptr(None), N.ptr(None), N.ptr(None), N.stream_ptr())
        N.check(rc, "ax_paged_decode_attention")
        return out
    outs = []
    G = Hq // Hkv
    for b in range(B):
        n = int(ctx_lens[b])
        pos = torch.arange(n, device=q.device)
        pages = block_table[b, (pos // page_size).long()].long()
        kk = k_cache[pages, (pos % page_size).long()].float().repeat_interleave(G, dim=1)   # [n, Hq, D]
        vv = v_cache[pages, (pos % page_size).long()].float().repeat_interleave(G, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), kk) * scale
        outs.append(torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vv))
    return torch.stack(outs).to(q.dtype)
