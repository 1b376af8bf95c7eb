"""Communication backends.

``Backend`` keeps the 13 methods of the reference's trait
(crates/axonml-distributed/src/backend.rs:87-126: name, rank, world_size, all_reduce, broadcast,
all_gather, reduce_scatter, gather, scatter, reduce, barrier, send, recv) but works on tensors of
any dtype on their own device, and every blocking call carries a timeout.  Implementations:

* ``MockBackend``   - in-process, for plumbing tests; ``create_world(n)`` returns n handles over
  one shared state (backend.rs:149-387).  Unlike the reference, a collective only completes when
  every rank has contributed (ranks are driven from threads), ``barrier`` really blocks, and a
  ``recv`` with no matching ``send`` raises after the timeout instead of silently doing nothing.
* ``CpuBackend``    - multi-process CPU ranks over ``torch.distributed`` gloo; runs the CPU DDP
  configuration and the failure-detection tests.
* ``NcclBackend``   - one process per GPU over NCCL / NVLink; the baseline transport, and the
  transport of pipeline send/recv.
"""
from __future__ import annotations

import datetime
import enum
import os
import threading
import time
from typing import Sequence

import torch
import torch.distributed as dist


class ReduceOp(enum.Enum):
    Sum = "sum"
    Product = "product"
    Min = "min"
    Max = "max"
    Average = "average"

    def apply_f32(self, a: float, b: float) -> float:
        if self is ReduceOp.Sum or self is ReduceOp.Average:
            return a + b
        if self is ReduceOp.Product:
            return a * b
        return min(a, b) if self is ReduceOp.Min else max(a, b)

    def reduce_slices(self, slices: Sequence[torch.Tensor]) -> torch.Tensor:
        st = torch.stack([s.to(torch.float32) if s.dtype in (torch.bfloat16, torch.float16) else s for s in slices])
        if self is ReduceOp.Sum: r = st.sum(0)
        elif self is ReduceOp.Average: r = st.sum(0) / len(slices)
        elif self is ReduceOp.Product: r = st.prod(0)
        elif self is ReduceOp.Min: r = st.min(0).values
        else: r = st.max(0).values
        return r.to(slices[0].dtype)

    def to_torch(self):
        return {ReduceOp.Sum: dist.ReduceOp.SUM, ReduceOp.Product: dist.ReduceOp.PRODUCT,
                ReduceOp.Min: dist.ReduceOp.MIN, ReduceOp.Max: dist.ReduceOp.MAX,
                ReduceOp.Average: dist.ReduceOp.AVG}[self]


class CommTimeout(RuntimeError):
    """A collective or point-to-point call did not complete within its timeout."""


class Backend:
    """Abstract transport.  All tensor arguments are modified in place where the reference's
    slices are (``all_reduce``, ``broadcast``); the others fill ``recv``."""

    timeout_s: float = 300.0

    def name(self) -> str: raise NotImplementedError
    def rank(self) -> int: raise NotImplementedError
    def world_size(self) -> int: raise NotImplementedError
    def all_reduce(self, data: torch.Tensor, op: ReduceOp = ReduceOp.Sum) -> None: raise NotImplementedError
    def broadcast(self, data: torch.Tensor, src: int = 0) -> None: raise NotImplementedError
    def all_gather(self, send: torch.Tensor, recv: torch.Tensor) -> None: raise NotImplementedError
    def reduce_scatter(self, send: torch.Tensor, recv: torch.Tensor, op: ReduceOp = ReduceOp.Sum) -> None: raise NotImplementedError
    def gather(self, send: torch.Tensor, recv: torch.Tensor | None, dst: int = 0) -> None: raise NotImplementedError
    def scatter(self, send: torch.Tensor | None, recv: torch.Tensor, src: int = 0) -> None: raise NotImplementedError
    def reduce(self, data: torch.Tensor, dst: int = 0, op: ReduceOp = ReduceOp.Sum) -> None: raise NotImplementedError
    def barrier(self) -> None: raise NotImplementedError

    def all_to_all(self, send: torch.Tensor, recv: torch.Tensor) -> None:
        """``send`` and ``recv`` are ``[world, ...]``: ``recv[j]`` receives rank j's ``send[rank]``.
        Generic form over ``all_gather``; transports with a native exchange override it."""
        w, r = self.world_size(), self.rank()
        full = torch.empty((w,) + tuple(send.shape), dtype=send.dtype, device=send.device)
        self.all_gather(send.contiguous(), full)
        recv.copy_(full[:, r])

    def send(self, data: torch.Tensor, dst: int, tag: int = 0) -> None: raise NotImplementedError
    def recv(self, data: torch.Tensor, src: int, tag: int = 0) -> None: raise NotImplementedError

    def sendrecv(self, send: torch.Tensor, dst: int, recv: torch.Tensor, src: int, tag: int = 0) -> None:
        """Sends to ``dst`` and receives from ``src`` in one step (a ring shift when every rank calls
        it).  Generic form for transports whose ``send`` does not wait for the receiver."""
        self.send(send, dst, tag)
        self.recv(recv, src, tag)

    def new_group(self, ranks: Sequence[int]) -> "Backend": raise NotImplementedError
    def device(self) -> torch.device: return torch.device("cpu")


# ------------------------------------------------------------------------------ mock
class _SharedState:
    def __init__(self, n: int):
        self.n = n
        self.cv = threading.Condition()
        self.rounds: dict = {}      # (kind, seq) -> {rank: tensor}
        self.results: dict = {}     # (kind, seq) -> (result, readers_left)
        self.messages: dict = {}    # (src, dst, tag) -> [tensor]
        self.dropped: set = set()   # fault injection: message keys to drop


class MockBackend(Backend):
    def __init__(self, rank: int, state: _SharedState, timeout_s: float = 5.0):
        self._rank, self._state, self.timeout_s = rank, state, timeout_s
        self._seq: dict = {}

    @classmethod
    def create_world(cls, n: int, timeout_s: float = 5.0) -> list:
        st = _SharedState(n)
        return [cls(r, st, timeout_s) for r in range(n)]

    @classmethod
    def single(cls) -> "MockBackend":
        return cls.create_world(1)[0]

    def name(self) -> str: return "mock"
    def rank(self) -> int: return self._rank
    def world_size(self) -> int: return self._state.n

    def _exchange(self, kind: str, value):
        """Deposits ``value`` and returns {rank: value} once all ranks have deposited."""
        st = self._state
        seq = self._seq.get(kind, 0)
        self._seq[kind] = seq + 1
        key = (kind, seq)
        deadline = time.monotonic() + self.timeout_s
        with st.cv:
            st.rounds.setdefault(key, {})[self._rank] = value
            if len(st.rounds[key]) == st.n:
                st.results[key] = [dict(st.rounds.pop(key)), st.n]
                st.cv.notify_all()
            while key not in st.results:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise CommTimeout(f"mock {kind} #{seq}: rank {self._rank} waited {self.timeout_s}s for the other ranks")
                st.cv.wait(left)
            res = st.results[key]
            res[1] -= 1
            out = res[0]
            if res[1] == 0:
                del st.results[key]
            return out

    def all_reduce(self, data, op=ReduceOp.Sum):
        parts = self._exchange("all_reduce", data.detach().clone())
        data.copy_(op.reduce_slices([parts[r] for r in range(self._state.n)]))

    def broadcast(self, data, src=0):
        parts = self._exchange("broadcast", data.detach().clone())
        data.copy_(parts[src])

    def all_gather(self, send, recv):
        parts = self._exchange("all_gather", send.detach().clone())
        recv.view(-1).copy_(torch.cat([parts[r].reshape(-1) for r in range(self._state.n)]))

    def reduce_scatter(self, send, recv, op=ReduceOp.Sum):
        parts = self._exchange("reduce_scatter", send.detach().clone())
        red = op.reduce_slices([parts[r].reshape(-1) for r in range(self._state.n)])
        n = recv.numel()
        recv.view(-1).copy_(red[self._rank * n:(self._rank + 1) * n])

    def gather(self, send, recv, dst=0):
        parts = self._exchange("gather", send.detach().clone())
        if self._rank == dst and recv is not None:
            recv.view(-1).copy_(torch.cat([parts[r].reshape(-1) for r in range(self._state.n)]))

    def scatter(self, send, recv, src=0):
        parts = self._exchange("scatter", send.detach().clone() if send is not None else None)
        n = recv.numel()
        recv.view(-1).copy_(parts[src].reshape(-1)[self._rank * n:(self._rank + 1) * n])

    def reduce(self, data, dst=0, op=ReduceOp.Sum):
        parts = self._exchange("reduce", data.detach().clone())
        if self._rank == dst:
            data.copy_(op.reduce_slices([parts[r] for r in range(self._state.n)]))

    def barrier(self):
        self._exchange("barrier", None)

    def send(self, data, dst, tag=0):
        st = self._state
        key = (self._rank, dst, tag)
        with st.cv:
            if key in st.dropped:
                st.dropped.discard(key)
                return
            st.messages.setdefault(key, []).append(data.detach().clone())
            st.cv.notify_all()

    def recv(self, data, src, tag=0):
        st = self._state
        key = (src, self._rank, tag)
        deadline = time.monotonic() + self.timeout_s
        with st.cv:
            while not st.messages.get(key):
                left = deadline - time.monotonic()
                if left <= 0:
                    raise CommTimeout(f"mock recv: rank {self._rank} got nothing from {src} (tag {tag}) in {self.timeout_s}s")
                st.cv.wait(left)
            data.copy_(st.messages[key].pop(0).reshape(data.shape))

    # fault injection (host side only)
    def drop_next_message(self, src: int, dst: int, tag: int = 0) -> None:
        with self._state.cv:
            self._state.dropped.add((src, dst, tag))

    def new_group(self, ranks):
        ranks = list(ranks)
        if self._rank not in ranks:
            return None
        key = ("group", tuple(ranks))
        with self._state.cv:
            sub = self._state.__dict__.setdefault("_subgroups", {})
            if key not in sub:
                sub[key] = _SharedState(len(ranks))
            st = sub[key]
        return MockBackend(ranks.index(self._rank), st, self.timeout_s)


# ------------------------------------------------------------------------------ torch.distributed
class _TorchDistBackend(Backend):
    """Shared implementation over a ``torch.distributed`` process group."""

    BACKEND = "gloo"

    def __init__(self, group=None, timeout_s: float = 300.0, _ranks=None):
        self.timeout_s = timeout_s
        self._group = group
        self._ranks = list(_ranks) if _ranks is not None else list(range(dist.get_world_size()))

    @classmethod
    def init(cls, rank: int | None = None, world_size: int | None = None,
             master_addr: str | None = None, master_port: int | None = None,
             timeout_s: float = 300.0, init_method: str | None = None):
        """Joins the job described by the arguments or by RANK / WORLD_SIZE / MASTER_ADDR /
        MASTER_PORT in the environment."""
        rank = int(os.environ.get("RANK", 0)) if rank is None else rank
        world_size = int(os.environ.get("WORLD_SIZE", 1)) if world_size is None else world_size
        if not dist.is_initialized():
            if init_method is None:
                addr = master_addr or os.environ.get("MASTER_ADDR", "127.0.0.1")
                port = master_port or int(os.environ.get("MASTER_PORT", 29500))
                init_method = f"tcp://{addr}:{port}"
            kwargs = {}
            if cls.BACKEND == "nccl":
                local = int(os.environ.get("LOCAL_RANK", rank % max(1, torch.cuda.device_count())))
                torch.cuda.set_device(local)
                kwargs["device_id"] = torch.device("cuda", local)
            dist.init_process_group(cls.BACKEND, init_method=init_method, rank=rank,
                                    world_size=world_size,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        return cls(None, timeout_s)

    def name(self) -> str: return self.BACKEND
    def rank(self) -> int: return dist.get_rank(self._group)
    def world_size(self) -> int: return dist.get_world_size(self._group)
    def group(self): return self._group
    def global_rank(self, group_rank: int) -> int: return self._ranks[group_rank]

    def _wrap(self, fn, what):
        try:
            return fn()
        except RuntimeError as e:  # gloo / nccl surface timeouts as RuntimeError
            msg = str(e)
            if "imeout" in msg or "timed out" in msg or "Connection closed" in msg or "reset by peer" in msg:
                raise CommTimeout(f"{self.BACKEND} {what}: {msg}") from e
            raise

    def all_reduce(self, data, op=ReduceOp.Sum):
        if op is ReduceOp.Average and self.BACKEND == "gloo":
            self._wrap(lambda: dist.all_reduce(data, dist.ReduceOp.SUM, self._group), "all_reduce")
            data.div_(self.world_size())
            return
        self._wrap(lambda: dist.all_reduce(data, op.to_torch(), self._group), "all_reduce")

    def broadcast(self, data, src=0):
        self._wrap(lambda: dist.broadcast(data, self._ranks[src], self._group), "broadcast")

    def all_gather(self, send, recv):
        self._wrap(lambda: dist.all_gather_into_tensor(recv.view(-1), send.contiguous().view(-1), self._group), "all_gather")

    def all_to_all(self, send, recv):
        if self.BACKEND == "gloo":
            return super().all_to_all(send, recv)
        self._wrap(lambda: dist.all_to_all_single(recv.view(-1), send.contiguous().view(-1), group=self._group), "all_to_all")

    def reduce_scatter(self, send, recv, op=ReduceOp.Sum):
        if self.BACKEND == "gloo":
            # gloo has no reduce_scatter: all_reduce a copy and keep this rank's slice
            tmp = send.detach().clone().view(-1)
            self.all_reduce(tmp, op)
            n = recv.numel()
            recv.view(-1).copy_(tmp[self.rank() * n:(self.rank() + 1) * n])
            return
        self._wrap(lambda: dist.reduce_scatter_tensor(recv.view(-1), send.contiguous().view(-1), op.to_torch(), self._group), "reduce_scatter")

    def gather(self, send, recv, dst=0):
        n = self.world_size()
        if self.BACKEND == "nccl" or True:
            tmp = torch.empty(n * send.numel(), dtype=send.dtype, device=send.device)
            self.all_gather(send, tmp)
            if self.rank() == dst and recv is not None:
                recv.view(-1).copy_(tmp)

    def scatter(self, send, recv, src=0):
        n = recv.numel()
        buf = send.contiguous().view(-1).clone() if (self.rank() == src and send is not None) else \
            torch.empty(n * self.world_size(), dtype=recv.dtype, device=recv.device)
        self.broadcast(buf, src)
        recv.view(-1).copy_(buf[self.rank() * n:(self.rank() + 1) * n])

    def reduce(self, data, dst=0, op=ReduceOp.Sum):
        if op is ReduceOp.Average:
            self._wrap(lambda: dist.reduce(data, self._ranks[dst], dist.ReduceOp.SUM, self._group), "reduce")
            if self.rank() == dst:
                data.div_(self.world_size())
            return
        self._wrap(lambda: dist.reduce(data, self._ranks[dst], op.to_torch(), self._group), "reduce")

    def barrier(self):
        self._wrap(lambda: dist.barrier(self._group), "barrier")

    def send(self, data, dst, tag=0):
        self._wrap(lambda: dist.send(data.contiguous(), self._ranks[dst], self._group, tag), "send")

    def recv(self, data, src, tag=0):
        self._wrap(lambda: dist.recv(data, self._ranks[src], self._group, tag), "recv")

    def sendrecv(self, send, dst, recv, src, tag=0):
        def go():
            ops = [dist.P2POp(dist.isend, send.contiguous(), self._ranks[dst], self._group, tag),
                   dist.P2POp(dist.irecv, recv, self._ranks[src], self._group, tag)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        self._wrap(go, "sendrecv")

    def isend(self, data, dst, tag=0): return dist.isend(data.contiguous(), self._ranks[dst], self._group, tag)
    def irecv(self, data, src, tag=0): return dist.irecv(data, self._ranks[src], self._group, tag)

    def new_group(self, ranks):
        ranks = list(ranks)
        g = dist.new_group([self._ranks[r] for r in ranks], timeout=datetime.timedelta(seconds=self.timeout_s))
        if self.rank() not in ranks:
            return None
        return type(self)(g, self.timeout_s, _ranks=[self._ranks[r] for r in ranks])

    def destroy(self) -> None:
        if dist.is_initialized() and self._group is None:
            dist.destroy_process_group()


class CpuBackend(_TorchDistBackend):
    BACKEND = "gloo"


class NcclBackend(_TorchDistBackend):
    BACKEND = "nccl"

    def device(self) -> torch.device:
        return torch.device("cuda", torch.cuda.current_device())


def init_from_env(timeout_s: float = 300.0) -> Backend:
    """NCCL when CUDA is available, gloo otherwise; single-process mock when WORLD_SIZE is unset."""
    if int(os.environ.get("WORLD_SIZE", "1")) <= 1 and not dist.is_initialized():
        return MockBackend.single()
    return (NcclBackend if torch.cuda.is_available() else CpuBackend).init(timeout_s=timeout_s)
