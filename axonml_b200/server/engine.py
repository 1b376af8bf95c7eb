"""LLM serving engine: request queue, continuous batching over a paged KV cache, greedy decoding,
time-to-first-token and decode-throughput accounting."""
from __future__ import annotations

import dataclasses
import itertools
import os
import time

import torch

from .kv_cache import PagedKVCache


@dataclasses.dataclass
class Request:
    rid: int
    prompt: list
    max_new_tokens: int
    eos_token_id: int | None = None
    arrival: float = 0.0
    first_token_at: float | None = None
    finished_at: float | None = None
    output: list = dataclasses.field(default_factory=list)
    slot: int = -1

    def ttft(self): return None if self.first_token_at is None else self.first_token_at - self.arrival
    def done(self) -> bool: return self.finished_at is not None


class LLMEngine:
    def __init__(self, model, max_batch: int = 64, max_context: int = 1024, page_size: int = 16,
                 num_pages: int | None = None):
        self.model, self.max_batch = model, max_batch
        if hasattr(model, "optimize_layout"):
            model.optimize_layout()
        cfg = model.cfg
        pages_per_seq = (max_context + page_size - 1) // page_size
        num_pages = num_pages or max_batch * pages_per_seq
        self.cache = PagedKVCache(cfg.num_hidden_layers, num_pages, page_size, model.hkv, model.hd, max_batch,
                                  pages_per_seq, model.device)
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self._ids = itertools.count()
        # CUDA-graph decode: one captured graph per batch size, fed through static input buffers
        self.use_graphs = model.device.type == "cuda" and os.environ.get("AXONML_DECODE_GRAPHS", "1") != "0"
        self._graphs: dict = {}
        if self.use_graphs:
            dev = model.device
            if model.tp > 1 and os.environ.get("AXONML_TP_COMM", "fused") == "nccl":
                # NCCL collectives are not captured here (a capture that stalls would stall every
                # rank until the process-group timeout): the NCCL variant decodes eagerly
                model.comm_mode = "nccl"
                self.use_graphs = False
            elif model.tp > 1:
                # create the peer-memory all-reduce now (a collective allocation, outside any capture);
                # without it the step would contain process-group calls, which are not captured
                model._all_reduce(torch.zeros(16, dtype=torch.bfloat16, device=dev))
                if not model._ar:
                    self.use_graphs = False
            self._g_tokens = torch.zeros(max_batch, dtype=torch.long, device=dev)
            self._g_slots = torch.zeros(max_batch, dtype=torch.int32, device=dev)
            self._g_pos = torch.zeros(max_batch, dtype=torch.int32, device=dev)
            self._g_next = torch.zeros(max_batch, dtype=torch.long, device=dev)
        self.decode_steps = 0
        self.decode_time = 0.0
        self.decode_tokens = 0
        self.prefill_time = 0.0

    def _now(self) -> float:
        if self.model.device.type == "cuda":
            torch.cuda.synchronize(self.model.device)
        return time.perf_counter()

    def add_request(self, prompt, max_new_tokens: int = 16, eos_token_id=None) -> Request:
        r = Request(next(self._ids), list(prompt), max_new_tokens, eos_token_id, time.perf_counter())
        self.waiting.append(r)
        return r

    def queue_depth(self) -> int: return len(self.waiting)

    # ------------------------------------------------------------------ one scheduler iteration
    @torch.no_grad()
    def step(self) -> None:
        admit = []
        if self.waiting and len(self.running) < self.max_batch:
            plen = len(self.waiting[0].prompt)
            for r in list(self.waiting):
                if len(r.prompt) != plen or len(self.running) + len(admit) >= self.max_batch:
                    break
                if not self.cache.can_admit(plen + r.max_new_tokens) and (admit or self.running):
                    break
                admit.append(r)
                self.waiting.remove(r)
        if admit:
            self._prefill(admit)
        elif self.running:
            self._decode()

    def _finish(self, r: Request, now: float) -> None:
        r.finished_at = now
        self.cache.free_seq(r.slot)
        self.running.remove(r)
        self.finished.append(r)

    def _prefill(self, reqs) -> None:
        t0 = self._now()
        for r in reqs:
            r.slot = self.cache.allocate_seq()
            self.cache.reserve(r.slot, len(r.prompt))
        ids = torch.tensor([r.prompt for r in reqs], dtype=torch.long, device=self.model.device)
        h = self.model.prefill(ids, self.cache, [r.slot for r in reqs])
        nxt = self.model.greedy(h).tolist()
        now = self._now()
        self.prefill_time += now - t0
        for r, t in zip(reqs, nxt):
            r.output.append(int(t))
            r.first_token_at = now
            self.running.append(r)
            if r.max_new_tokens <= 1 or t == r.eos_token_id:
                self._finish(r, now)

    def _decode(self) -> None:
        t0 = self._now()
        reqs = list(self.running)
        dev = self.model.device
        pos = [len(r.prompt) + len(r.output) - 1 for r in reqs]
        for r, p in zip(reqs, pos):
            self.cache.reserve(r.slot, p + 1)
        tokens = torch.tensor([r.output[-1] for r in reqs], dtype=torch.long, device=dev)
        slots = torch.tensor([r.slot for r in reqs], dtype=torch.int32, device=dev)
        positions = torch.tensor(pos, dtype=torch.int32, device=dev)
        nxt = self._decode_step(tokens, slots, positions).tolist()
        now = self._now()
        self.decode_time += now - t0
        self.decode_steps += 1
        self.decode_tokens += len(reqs)
        for r, t in zip(reqs, nxt):
            r.output.append(int(t))
            if len(r.output) >= r.max_new_tokens or t == r.eos_token_id:
                self._finish(r, now)

    def _decode_step(self, tokens, slots, positions) -> torch.Tensor:
        """Eager decode, or replay of the CUDA graph captured for this batch size (the whole step -
        embedding gather, 32 layers, head, arg-max - is one graph launch, which removes the
        per-kernel launch overhead that dominates small-batch decoding)."""
        B = tokens.shape[0]
        if not self.use_graphs:
            return self.model.greedy(self.model.decode(tokens, self.cache, slots, positions))
        self._g_tokens[:B].copy_(tokens)
        self._g_slots[:B].copy_(slots)
        self._g_pos[:B].copy_(positions)
        g = self._graphs.get(B)
        if g is None:
            def run():
                h = self.model.decode(self._g_tokens[:B], self.cache, self._g_slots[:B], self._g_pos[:B])
                self._g_next[:B].copy_(self.model.greedy(h))
            side = torch.cuda.Stream(self.model.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):        # warm-up outside capture (lazy initialisation, attributes)
                run()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                run()
            self._graphs[B] = g
            # the warm-up and the capture both ran the step on real inputs; replaying once more
            # rewrites the same K/V rows, so the result is unchanged
        g.replay()
        return self._g_next[:B].clone()

    def warmup(self, batch_sizes=None) -> None:
        """Captures the decode graphs ahead of the first request (server start-up), so no request
        pays for a capture.  Uses scratch sequences of one token that are freed afterwards."""
        if not self.use_graphs or self.running or self.waiting:
            return
        sizes = sorted(set(batch_sizes or [1, 2, 4, 8, 16, 32, self.max_batch]))
        dev = self.model.device
        for B in sizes:
            if B in self._graphs or B > self.max_batch:
                continue
            slots = [self.cache.allocate_seq() for _ in range(B)]
            for sl in slots:
                self.cache.reserve(sl, 1)
            self._decode_step(torch.zeros(B, dtype=torch.long, device=dev),
                              torch.tensor(slots, dtype=torch.int32, device=dev),
                              torch.zeros(B, dtype=torch.int32, device=dev))
            for sl in slots:
                self.cache.free_seq(sl)
        torch.cuda.synchronize(dev)

    def run_until_done(self) -> None:
        while self.waiting or self.running:
            self.step()

    def generate(self, prompts, max_new_tokens: int = 16, eos_token_id=None) -> list:
        reqs = [self.add_request(p, max_new_tokens, eos_token_id) for p in prompts]
        self.run_until_done()
        return [r.output for r in reqs]

    def stats(self) -> dict:
        ttfts = sorted(r.ttft() for r in self.finished if r.ttft() is not None)
        p50 = ttfts[len(ttfts) // 2] if ttfts else None
        return {"requests": len(self.finished), "ttft_p50_s": p50,
                "decode_tokens_per_s": self.decode_tokens / self.decode_time if self.decode_time else 0.0,
                "decode_steps": self.decode_steps, "decode_time_s": self.decode_time, "prefill_time_s": self.prefill_time,
                "kv_page_occupancy": self.cache.occupancy(), "queue_depth": self.queue_depth()}
