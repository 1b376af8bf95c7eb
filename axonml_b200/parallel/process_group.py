"""ProcessGroup and World (crates/axonml-distributed/src/process_group.rs:18-204).  Tensor-level
collectives keep the reference's shapes: ``all_gather_tensor`` returns ``[world, *shape]``,
``reduce_scatter_tensor`` splits dim 0 by the world size.  Sub-groups are real communicators (the
reference stores a rank list that its collectives ignore, process_group.rs:34-36)."""
from __future__ import annotations

from typing import Sequence

import torch

from .backend import Backend, MockBackend, ReduceOp


class ProcessGroup:
    def __init__(self, backend: Backend, ranks: Sequence[int] | None = None):
        self._backend = backend
        self._ranks = list(ranks) if ranks is not None else list(range(backend.world_size()))

    @classmethod
    def new(cls, backend): return cls(backend)

    @classmethod
    def with_ranks(cls, backend: Backend, ranks: Sequence[int]):
        sub = backend.new_group(ranks)
        return cls(sub if sub is not None else backend, ranks)

    @classmethod
    def mock(cls): return cls(MockBackend.single())

    def backend(self) -> Backend: return self._backend
    def rank(self) -> int: return self._backend.rank()
    def world_size(self) -> int: return self._backend.world_size()
    def size(self) -> int: return self.world_size()
    def ranks(self): return list(self._ranks)
    def contains(self, rank: int) -> bool: return rank in self._ranks
    def barrier(self) -> None: self._backend.barrier()

    def all_reduce_tensor(self, t: torch.Tensor, op: ReduceOp = ReduceOp.Sum) -> torch.Tensor:
        self._backend.all_reduce(t, op)
        return t

    def broadcast_tensor(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        self._backend.broadcast(t, src)
        return t

    def all_gather_tensor(self, t: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.world_size(),) + tuple(t.shape), dtype=t.dtype, device=t.device)
        self._backend.all_gather(t.contiguous(), out)
        return out

    def reduce_scatter_tensor(self, t: torch.Tensor, op: ReduceOp = ReduceOp.Sum) -> torch.Tensor:
        w = self.world_size()
        if t.shape[0] % w:
            raise ValueError("dim 0 must be divisible by the world size")
        out = torch.empty((t.shape[0] // w,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        self._backend.reduce_scatter(t.contiguous(), out, op)
        return out

    def send_tensor(self, t: torch.Tensor, dst: int, tag: int = 0) -> None:
        self._backend.send(t, dst, tag)

    def recv_tensor(self, src: int, shape, tag: int = 0, dtype=torch.float32, device=None) -> torch.Tensor:
        out = torch.empty(tuple(shape), dtype=dtype, device=device or self._backend.device())
        self._backend.recv(out, src, tag)
        return out


class World:
    def __init__(self, backend: Backend):
        self._backend = backend
        self._default = ProcessGroup(backend)

    @classmethod
    def init(cls, backend: Backend): return cls(backend)

    @classmethod
    def mock(cls): return cls(MockBackend.single())

    @classmethod
    def from_env(cls, timeout_s: float = 300.0):
        from .backend import init_from_env
        return cls(init_from_env(timeout_s))

    def default_group(self) -> ProcessGroup: return self._default
    def rank(self) -> int: return self._backend.rank()
    def world_size(self) -> int: return self._backend.world_size()
    def is_main(self) -> bool: return self.rank() == 0
    def barrier(self) -> None: self._backend.barrier()
    def new_group(self, ranks) -> ProcessGroup: return ProcessGroup.with_ranks(self._backend, ranks)
    def backend(self) -> Backend: return self._backend
