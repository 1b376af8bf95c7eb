"""Quantised LLaMA for serving: Q4_K projection weights, Q8_0 embedding and output head, bf16
paged KV cache, tensor parallel over the process group (heads and FFN columns split across ranks,
vocabulary-parallel head).  Weights come from a GGUF file or are drawn N(0, 0.02) and quantised on
the GPU (``from_random``).

Every projection is the fused dequantising matmul (``ops.quant.qlinear``); prefill attention is
the flash kernel, decode attention reads the paged cache; the two all-reduces per layer use the
fused peer-memory all-reduce kernel when symmetric memory is available, NCCL otherwise."""
from __future__ import annotations

import math

import torch

from ..llm.config import LLaMAConfig
from ..ops import elementwise as E
from ..ops import misc as Mi
from ..ops import norm as Nm
from ..ops import paged
from ..ops.attention import sdpa
from ..ops.quant import qlinear
from ..quant.quantize import dequantize_tensor, quantize_tensor
from ..quant.types import QuantizedTensor, QuantType


class _Layer:
    __slots__ = ("attn_norm", "wqkv", "wo", "ffn_norm", "wgu", "wdown")


class QuantizedLlama:
    def __init__(self, cfg: LLaMAConfig, pg=None, device="cuda"):
        self.cfg, self.pg, self.device = cfg, pg, torch.device(device)
        self.tp = pg.world_size() if pg is not None else 1
        self.rank = pg.rank() if pg is not None else 0
        if cfg.num_attention_heads % self.tp or cfg.num_key_value_heads % self.tp or cfg.intermediate_size % self.tp:
            raise ValueError("heads / kv heads / FFN width must be divisible by the tensor-parallel size")
        self.hq, self.hkv, self.hd = cfg.num_attention_heads // self.tp, cfg.num_key_value_heads // self.tp, cfg.head_dim()
        self.ffn = cfg.intermediate_size // self.tp
        self.vocab_local = (cfg.vocab_size + self.tp - 1) // self.tp
        self.layers: list[_Layer] = []
        self.embed = None
        self.head = None
        self.final_norm = None
        cos, sin = Mi.rope_tables(cfg.max_position_embeddings, self.hd, cfg.rope_theta, device=self.device)
        self.cos, self.sin = cos, sin
        self._ar = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_random(cls, cfg: LLaMAConfig, pg=None, device="cuda", seed: int = 0, std: float = 0.02,
                    proj_type: QuantType = QuantType.Q4_K):
        m = cls(cfg, pg, device)
        g = torch.Generator(device=m.device).manual_seed(seed + 1000 * m.rank)
        H = cfg.hidden_size

        def rnd(rows, cols, qt):
            w = torch.empty(rows, cols, device=m.device, dtype=torch.float32).normal_(0.0, std, generator=g)
            return quantize_tensor(w, qt)
        for _ in range(cfg.num_hidden_layers):
            L = _Layer()
            L.attn_norm = torch.ones(H, device=m.device, dtype=torch.bfloat16)
            L.ffn_norm = torch.ones(H, device=m.device, dtype=torch.bfloat16)
            L.wqkv = rnd((m.hq + 2 * m.hkv) * m.hd, H, proj_type)
            L.wo = rnd(H, m.hq * m.hd, proj_type)
            L.wgu = rnd(2 * m.ffn, H, proj_type)
            L.wdown = rnd(H, m.ffn, proj_type)
            m.layers.append(L)
        m.embed = rnd(cfg.vocab_size, H, QuantType.Q8_0)
        m.head = rnd(m.vocab_local, H, QuantType.Q8_0)
        m.final_norm = torch.ones(H, device=m.device, dtype=torch.bfloat16)
        return m

    @classmethod
    def from_gguf(cls, path, pg=None, device="cuda"):
        from ..quant.gguf import read_gguf
        g = read_gguf(path)
        md = g.metadata
        a = md.get("general.architecture", "llama")
        cfg = LLaMAConfig(vocab_size=int(md.get(f"{a}.vocab_size", g.tensors["token_embd.weight"][0][0])),
                          hidden_size=int(md[f"{a}.embedding_length"]), intermediate_size=int(md[f"{a}.feed_forward_length"]),
                          num_hidden_layers=int(md[f"{a}.block_count"]), num_attention_heads=int(md[f"{a}.attention.head_count"]),
                          num_key_value_heads=int(md.get(f"{a}.attention.head_count_kv", md[f"{a}.attention.head_count"])),
                          max_position_embeddings=int(md.get(f"{a}.context_length", 4096)),
                          rms_norm_eps=float(md.get(f"{a}.attention.layer_norm_rms_epsilon", 1e-5)),
                          rope_theta=float(md.get(f"{a}.rope.freq_base", 10000.0)))
        m = cls(cfg, pg, device)
        tp, r, hd = m.tp, m.rank, m.hd

        def rows(name, lo, hi, qt_fallback=QuantType.Q4_K):
            """Rows [lo, hi) of a 2-D GGUF tensor, kept quantised when its blocks do not straddle rows."""
            shape, qt, _, _ = g.tensors[name]
            q = g.quantized(name)
            if qt.is_block_quantized() and shape[1] % qt.block_size() == 0:
                rb = shape[1] // qt.block_size() * qt.bytes_per_block()
                return QuantizedTensor([hi - lo, shape[1]], qt, q.data[lo * rb:hi * rb].to(m.device))
            w = dequantize_tensor(q)[lo:hi].to(m.device)
            return quantize_tensor(w, qt_fallback if w.shape[1] % 256 == 0 else QuantType.Q8_0)

        def cols(name, lo, hi):
            """Columns [lo, hi) of a 2-D GGUF tensor.  Blocks run along the columns, so a slice on
            block boundaries is a byte slice of every row: the quantised values are kept exactly."""
            shape, qt, _, _ = g.tensors[name]
            if qt.is_block_quantized() and shape[1] % qt.block_size() == 0 and lo % qt.block_size() == 0 \
                    and hi % qt.block_size() == 0:
                q = g.quantized(name)
                bs, bb = qt.block_size(), qt.bytes_per_block()
                d = q.data.view(shape[0], shape[1] // bs, bb)[:, lo // bs:hi // bs].contiguous()
                return QuantizedTensor([shape[0], hi - lo], qt, d.view(-1).to(m.device))
            w = g.tensor(name)[:, lo:hi].contiguous().to(m.device)
            return quantize_tensor(w, QuantType.Q4_K if w.shape[1] % 256 == 0 else QuantType.Q8_0)

        def cat(parts):
            return QuantizedTensor([sum(p.shape[0] for p in parts), parts[0].shape[1]], parts[0].quant_type,
                                   torch.cat([p.data for p in parts]))
        for i in range(cfg.num_hidden_layers):
            L, p = _Layer(), f"blk.{i}."
            L.attn_norm = g.tensor(p + "attn_norm.weight").to(m.device, torch.bfloat16)
            L.ffn_norm = g.tensor(p + "ffn_norm.weight").to(m.device, torch.bfloat16)
            nq, nk = m.hq * hd, m.hkv * hd
            parts = [rows(p + "attn_q.weight", r * nq, (r + 1) * nq), rows(p + "attn_k.weight", r * nk, (r + 1) * nk),
                     rows(p + "attn_v.weight", r * nk, (r + 1) * nk)]
            if len({x.quant_type for x in parts}) > 1:
                parts = [quantize_tensor(dequantize_tensor(x), QuantType.Q4_K) for x in parts]
            L.wqkv = cat(parts)
            L.wo = cols(p + "attn_output.weight", r * nq, (r + 1) * nq) if tp > 1 else rows(p + "attn_output.weight", 0, cfg.hidden_size)
            gu = [rows(p + "ffn_gate.weight", r * m.ffn, (r + 1) * m.ffn), rows(p + "ffn_up.weight", r * m.ffn, (r + 1) * m.ffn)]
            if gu[0].quant_type != gu[1].quant_type:
                gu = [quantize_tensor(dequantize_tensor(x), QuantType.Q4_K) for x in gu]
            L.wgu = cat(gu)
            L.wdown = cols(p + "ffn_down.weight", r * m.ffn, (r + 1) * m.ffn) if tp > 1 else rows(p + "ffn_down.weight", 0, cfg.hidden_size)
            m.layers.append(L)
        m.embed = rows("token_embd.weight", 0, cfg.vocab_size, QuantType.Q8_0)
        hn = "output.weight" if "output.weight" in g.tensors else "token_embd.weight"
        lo = r * m.vocab_local
        m.head = rows(hn, lo, min(cfg.vocab_size, lo + m.vocab_local), QuantType.Q8_0)
        m.final_norm = g.tensor("output_norm.weight").to(m.device, torch.bfloat16)
        g.close()
        return m

    def to_gguf(self, path) -> None:
        """Writes this rank's weights as a GGUF file (single-rank models are complete checkpoints)."""
        from ..quant.gguf import write_gguf
        c, hd = self.cfg, self.hd
        t, nq, nk = {}, self.hq * hd, self.hkv * hd

        def part(q: QuantizedTensor, lo, hi):
            rb = q.shape[1] // q.quant_type.block_size() * q.quant_type.bytes_per_block()
            return QuantizedTensor([hi - lo, q.shape[1]], q.quant_type, q.data[lo * rb:hi * rb])
        for i, L in enumerate(self.layers):
            p = f"blk.{i}."
            t[p + "attn_norm.weight"], t[p + "ffn_norm.weight"] = L.attn_norm.float(), L.ffn_norm.float()
            t[p + "attn_q.weight"], t[p + "attn_k.weight"] = part(L.wqkv, 0, nq), part(L.wqkv, nq, nq + nk)
            t[p + "attn_v.weight"], t[p + "attn_output.weight"] = part(L.wqkv, nq + nk, nq + 2 * nk), L.wo
            t[p + "ffn_gate.weight"], t[p + "ffn_up.weight"] = part(L.wgu, 0, self.ffn), part(L.wgu, self.ffn, 2 * self.ffn)
            t[p + "ffn_down.weight"] = L.wdown
        t["token_embd.weight"], t["output.weight"], t["output_norm.weight"] = self.embed, self.head, self.final_norm.float()
        md = {"general.architecture": "llama", "general.name": "axonml-llama", "llama.vocab_size": c.vocab_size,
              "llama.embedding_length": c.hidden_size, "llama.feed_forward_length": c.intermediate_size,
              "llama.block_count": c.num_hidden_layers, "llama.attention.head_count": c.num_attention_heads,
              "llama.attention.head_count_kv": c.num_key_value_heads, "llama.context_length": c.max_position_embeddings,
              "llama.attention.layer_norm_rms_epsilon": float(c.rms_norm_eps), "llama.rope.freq_base": float(c.rope_theta)}
        write_gguf(path, t, md)

    def optimize_layout(self) -> "QuantizedLlama":
        """Repacks the projection weights and the head into the tile layout of the dequantising
        matmul (GPU only).  Prefill of long prompts dequantises from the same data."""
        if self.device.type != "cuda":
            return self
        from ..ops.quant import tile_weight
        ok = lambda q: q.layout == "ggml" and q.quant_type in (QuantType.Q4_K, QuantType.Q8_0) and q.shape[1] % 256 == 0
        for L in self.layers:
            for name in ("wqkv", "wo", "wgu", "wdown"):
                q = getattr(L, name)
                if ok(q):
                    setattr(L, name, tile_weight(q))
        if ok(self.head):
            self.head = tile_weight(self.head)
        return self

    def weight_bytes(self) -> int:
        n = self.embed.size_bytes() + self.head.size_bytes()
        for L in self.layers:
            n += L.wqkv.size_bytes() + L.wo.size_bytes() + L.wgu.size_bytes() + L.wdown.size_bytes()
        return n

    # ------------------------------------------------------------------ forward
    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over the tensor-parallel ranks.  On GPUs this is the one-launch all-reduce kernel over
        peer memory with its call counter on the device, so decode steps that contain it can be
        captured in CUDA graphs; elsewhere (CPU ranks, no symmetric memory) the process group's
        all-reduce."""
        if self.tp == 1:
            return x
        if self._ar is None:
            self._ar = False
            if x.is_cuda and getattr(self, "comm_mode", "fused") != "nccl":
                from ..parallel.fused import FusedAllReduce
                self._ar = FusedAllReduce.try_create(self.pg, 64 * 512 * self.cfg.hidden_size, torch.bfloat16,
                                                     device_epoch=True) or False
                self._ar32 = FusedAllReduce.try_create(self.pg, 4096, torch.float32, device_epoch=True) if self._ar else None
        if self._ar and x.dtype == torch.bfloat16 and x.numel() <= self._ar.capacity:
            flat = x.reshape(-1)
            if x.is_contiguous() and self._ar.sum_small_(flat):          # decode-sized vectors: one trip, no staging copy
                return x
            self._ar.all_reduce_mean_(flat)
            return x.mul_(self.tp)
        from ..parallel.backend import ReduceOp
        self.pg.backend().all_reduce(x, ReduceOp.Sum)
        return x

    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        rb = self.cfg.hidden_size // 32 * 34
        rows = self.embed.data.view(-1, rb)[ids.reshape(-1).long()]
        q = QuantizedTensor([rows.shape[0], self.cfg.hidden_size], self.embed.quant_type, rows.reshape(-1))
        if q.quant_type is not QuantType.Q8_0:
            raise ValueError("token embedding must be Q8_0")
        return dequantize_tensor(q, torch.bfloat16)

    def _logits(self, h: torch.Tensor) -> torch.Tensor:
        from ..ops import decode as Dc
        if (h.dim() == 2 and h.shape[0] <= 4 and h.is_contiguous() and Dc.supported(h)
                and Dc.gemv_ok(self.head, h.shape[0])):
            a, _, _ = Dc.rms_norm_q8(h, self.final_norm, self.cfg.rms_norm_eps)     # norm -> int8 for the head kernel
            return Dc.qgemv(a, self.head, out_dtype=torch.float32)
        return qlinear(Nm.rms_norm(h, self.final_norm, self.cfg.rms_norm_eps), self.head, out_dtype=torch.float32)

    def greedy(self, h: torch.Tensor) -> torch.Tensor:
        """Next token per row of ``h`` with the vocabulary split over ranks: local arg-max, then one
        tiny all-gather of (value, index) pairs."""
        lg = self._logits(h)
        V = lg.shape[-1]
        if V >= 65536 and V % 256 == 0:
            # two stages: a single-row reduction over the whole vocabulary runs in one thread block
            v1, i1 = lg.view(-1, 256, V // 256).max(dim=-1)
            val, i2 = v1.max(dim=-1)
            idx = i2 * (V // 256) + i1.gather(-1, i2.unsqueeze(-1)).squeeze(-1)
        else:
            val, idx = lg.max(dim=-1)
        idx = idx + self.rank * self.vocab_local
        if self.tp == 1:
            return idx
        pair = torch.stack([val, idx.float()], dim=-1).contiguous()
        ar32 = getattr(self, "_ar32", None) if self._ar else None
        if ar32 is not None and self.tp * pair.numel() <= ar32.capacity:
            # every rank writes its pairs into its own slot of a zero buffer; the sum is the gather
            # (graph-capturable, unlike the process group's all-gather)
            out = torch.zeros((self.tp,) + tuple(pair.shape), dtype=pair.dtype, device=pair.device)
            out[self.rank] = pair
            if not ar32.sum_small_(out.view(-1)):
                ar32.all_reduce_mean_(out.view(-1))
                out = out * self.tp
        else:
            out = torch.empty((self.tp,) + tuple(pair.shape), dtype=pair.dtype, device=pair.device)
            self.pg.backend().all_gather(pair, out)
        best = out[..., 0].argmax(dim=0)
        return out[..., 1].gather(0, best.unsqueeze(0)).squeeze(0).round().long()

    def prefill(self, ids: torch.Tensor, cache, slots, layer_write=True) -> torch.Tensor:
        """``ids`` [B, S] (equal-length prompts); writes K/V of every token into the pages of
        ``slots`` and returns the hidden state of the last token of each prompt, [B, H]."""
        B, S = ids.shape
        x = self._embed(ids).view(B * S, -1)
        seq = torch.tensor(slots, dtype=torch.int32, device=self.device).repeat_interleave(S)
        pos = torch.arange(S, dtype=torch.int32, device=self.device).repeat(B)
        nq, nk = self.hq * self.hd, self.hkv * self.hd
        for li, L in enumerate(self.layers):
            h = Nm.rms_norm(x, L.attn_norm, self.cfg.rms_norm_eps)
            qkv = qlinear(h, L.wqkv).view(B * S, self.hq + 2 * self.hkv, self.hd)
            qkv = Mi.rope_positions(qkv, self.cos, self.sin, pos, rot_heads=self.hq + self.hkv)
            q, k, v = qkv[:, :self.hq], qkv[:, self.hq:self.hq + self.hkv], qkv[:, self.hq + self.hkv:]
            paged.kv_write(k, v, cache.k[li], cache.v[li], cache.block_table, seq, pos, cache.page_size)
            a = sdpa(q.reshape(B, S, self.hq, self.hd), k.reshape(B, S, self.hkv, self.hd),
                     v.reshape(B, S, self.hkv, self.hd), causal=True)
            o = self._all_reduce(qlinear(a.reshape(B * S, nq), L.wo))
            x = x + o
            h = Nm.rms_norm(x, L.ffn_norm, self.cfg.rms_norm_eps)
            d = self._all_reduce(qlinear(E.swiglu(qlinear(h, L.wgu)), L.wdown))
            x = x + d
        return x.view(B, S, -1)[:, -1]

    def _fused_decode_ok(self, B: int, cache) -> bool:
        """Batches of up to four rows on the matrix-vector kernels: every producer writes int8
        activations itself and RoPE + KV write are one launch (``ops/decode.py``)."""
        import os
        from ..ops import decode as Dc
        if os.environ.get("AXONML_DECODE_FUSED", "1") == "0" or self.hd != 128 or not self.layers:
            return False
        from .. import _native as N
        L = self.layers[0]
        return (N.is_blackwell() and self.device.type == "cuda" and self.cfg.hidden_size % 32 == 0 and self.ffn % 32 == 0
                and self.hq // self.hkv in (1, 2, 4, 8)
                and all(Dc.gemv_ok(w, B) for w in (L.wqkv, L.wo, L.wgu, L.wdown)))

    def _decode_fused(self, tokens, cache, slots_t, positions) -> torch.Tensor:
        """The decode step with ten launches per layer: qkv product, rope + q copy + KV write,
        attention (split and merge, the merge writing int8), o product, add + norm -> int8, gate|up
        product, SwiGLU -> int8, down product, add + norm -> int8."""
        from ..ops import decode as Dc
        B = tokens.shape[0]
        eps = self.cfg.rms_norm_eps
        x = self._embed(tokens)
        ctx = positions + 1
        table = cache.block_table[slots_t.long()].contiguous()
        seq_local = torch.arange(B, dtype=torch.int32, device=self.device)
        a, x, _ = Dc.rms_norm_q8(x, self.layers[0].attn_norm, eps)
        for li, L in enumerate(self.layers):
            qkv = Dc.qgemv(a, L.wqkv).view(B, self.hq + 2 * self.hkv, self.hd)
            q = Dc.rope_kv_write(qkv, self.cos, self.sin, positions, cache.k[li], cache.v[li], table, seq_local,
                                 self.hq, self.hkv, cache.page_size)
            _, a = Dc.decode_attention_q8(q, cache.k[li], cache.v[li], table, ctx, cache.page_size)
            o = self._all_reduce(Dc.qgemv(a, L.wo))
            a, x, _ = Dc.rms_norm_q8(x, L.ffn_norm, eps, residual=o)
            a = Dc.swiglu_q8(Dc.qgemv(a, L.wgu))
            d = self._all_reduce(Dc.qgemv(a, L.wdown))
            if li + 1 < len(self.layers):
                a, x, _ = Dc.rms_norm_q8(x, self.layers[li + 1].attn_norm, eps, residual=d)
            else:
                x = x + d
        return x

    def decode(self, tokens: torch.Tensor, cache, slots_t: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One token per running sequence.  ``tokens`` [B], ``slots_t`` [B] int32 cache slots,
        ``positions`` [B] int32 position of the new token.  Returns the hidden state [B, H]."""
        B = tokens.shape[0]
        if B <= 4 and self._fused_decode_ok(B, cache):
            return self._decode_fused(tokens, cache, slots_t, positions)
        x = self._embed(tokens)
        ctx = positions + 1
        table = cache.block_table[slots_t.long()]
        seq_local = torch.arange(B, dtype=torch.int32, device=self.device)
        nq = self.hq * self.hd
        h = Nm.rms_norm(x, self.layers[0].attn_norm, self.cfg.rms_norm_eps)
        for li, L in enumerate(self.layers):
            qkv = qlinear(h, L.wqkv).view(B, self.hq + 2 * self.hkv, self.hd)
            qkv = Mi.rope_positions(qkv, self.cos, self.sin, positions, rot_heads=self.hq + self.hkv)
            q, k, v = qkv[:, :self.hq], qkv[:, self.hq:self.hq + self.hkv], qkv[:, self.hq + self.hkv:]
            paged.kv_write(k, v, cache.k[li], cache.v[li], table, seq_local, positions, cache.page_size)
            a = paged.decode_attention(q.contiguous(), cache.k[li], cache.v[li], table, ctx, cache.page_size)
            o = self._all_reduce(qlinear(a.reshape(B, nq), L.wo))
            h, x = Nm.rms_norm(o, L.ffn_norm, self.cfg.rms_norm_eps, residual=x)     # x += o, fused
            d = self._all_reduce(qlinear(E.swiglu(qlinear(h, L.wgu)), L.wdown))
            if li + 1 < len(self.layers):
                h, x = Nm.rms_norm(d, self.layers[li + 1].attn_norm, self.cfg.rms_norm_eps, residual=x)
            else:
                x = x + d
        return x
