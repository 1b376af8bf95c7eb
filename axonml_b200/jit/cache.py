"""Compiled-function cache keyed by a structural graph hash (crates/axonml-jit/src/cache.rs:14-212)."""
from __future__ import annotations

import collections
import dataclasses
import hashlib
import threading


@dataclasses.dataclass
class CacheStats:
    entries: int
    max_size: int
    hits: int = 0
    misses: int = 0

    def utilization(self) -> float: return self.entries / self.max_size if self.max_size else 0.0


class FunctionCache:
    def __init__(self, max_size: int = 1000):
        self.max_size = max_size
        self._d: collections.OrderedDict = collections.OrderedDict()
        self._lock = threading.Lock()
        self.hits = self.misses = 0

    @classmethod
    def new(cls, max_size): return cls(max_size)
    @classmethod
    def default_size(cls): return cls(1000)

    @staticmethod
    def hash_graph(graph) -> int:
        return int.from_bytes(hashlib.blake2b(repr(graph.signature()).encode(), digest_size=8).digest(), "little")

    def get(self, key: int):
        with self._lock:
            f = self._d.get(key)
            if f is None:
                self.misses += 1
            else:
                self.hits += 1
                self._d.move_to_end(key)
            return f

    def get_by_graph(self, graph): return self.get(self.hash_graph(graph))

    def insert(self, key: int, func) -> None:
        with self._lock:
            self._d[key] = func
            self._d.move_to_end(key)
            while len(self._d) > self.max_size:
                self._d.popitem(last=False)

    def insert_for_graph(self, graph, func): self.insert(self.hash_graph(graph), func)
    def len(self) -> int: return len(self._d)
    def __len__(self) -> int: return len(self._d)
    def is_empty(self) -> bool: return not self._d
    def clear(self) -> None:
        with self._lock:
            self._d.clear()
    def stats(self) -> CacheStats: return CacheStats(len(self._d), self.max_size, self.hits, self.misses)
