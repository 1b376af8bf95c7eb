"""Paged KV cache: a pool of fixed-size pages per layer plus a block table per sequence
(replaces the reference's concat-and-grow ``KVCache``, crates/axonml-llm/src/attention.rs:19-86)."""
from __future__ import annotations

import torch


class OutOfPages(RuntimeError):
    pass


class PagedKVCache:
    def __init__(self, num_layers: int, num_pages: int, page_size: int, num_kv_heads: int, head_dim: int,
                 max_seqs: int, max_pages_per_seq: int, device, dtype=torch.bfloat16):
        self.num_layers, self.num_pages, self.page_size = num_layers, num_pages, page_size
        self.max_seqs, self.max_pages_per_seq = max_seqs, max_pages_per_seq
        shape = (num_layers, num_pages, page_size, num_kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.block_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=device)
        self._table_host = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32)
        self._free_pages = list(range(num_pages - 1, -1, -1))
        self._free_slots = list(range(max_seqs - 1, -1, -1))
        self._pages_of: dict[int, list] = {}
        self.lens: dict[int, int] = {}

    def pages_free(self) -> int: return len(self._free_pages)
    def occupancy(self) -> float: return 1.0 - len(self._free_pages) / self.num_pages
    def can_admit(self, tokens: int) -> bool:
        return bool(self._free_slots) and (tokens + self.page_size - 1) // self.page_size <= len(self._free_pages)

    def allocate_seq(self) -> int:
        if not self._free_slots:
            raise OutOfPages("no free sequence slot")
        s = self._free_slots.pop()
        self._pages_of[s], self.lens[s] = [], 0
        return s

    def reserve(self, slot: int, new_len: int) -> None:
        """Makes sure ``slot`` owns enough pages for ``new_len`` tokens."""
        need = (new_len + self.page_size - 1) // self.page_size
        pages = self._pages_of[slot]
        if need > self.max_pages_per_seq:
            raise OutOfPages("sequence exceeds the maximum context")
        changed = False
        while len(pages) < need:
            if not self._free_pages:
                raise OutOfPages("KV cache is full")
            p = self._free_pages.pop()
            self._table_host[slot, len(pages)] = p
            pages.append(p)
            changed = True
        if changed:
            self.block_table[slot].copy_(self._table_host[slot], non_blocking=True)
        self.lens[slot] = new_len

    def free_seq(self, slot: int) -> None:
        self._free_pages.extend(reversed(self._pages_of.pop(slot, [])))
        self.lens.pop(slot, None)
        self._free_slots.append(slot)
