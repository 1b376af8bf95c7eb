"""Flat-parameter unit of the fully-sharded engine.

A unit owns a set of parameters laid out back to back (each start aligned to 64 elements, so that
every parameter can be a TMA source) in one flat low-precision buffer.  The flat range is padded
to a multiple of the world size and split evenly: rank r owns elements
``[r*shard, (r+1)*shard)``, which is the reference's ``ceil(numel/world)`` zero-padded shard rule
(crates/axonml-distributed/src/fsdp.rs:168-212) applied per unit.

Per rank a unit holds: the fp32 master shard (a leaf ``Parameter`` that the optimizer steps), a
low-precision shard that the optimizer kernel refreshes, the flat gradient buffer that backward
fills, and the reduced gradient shard.
"""
from __future__ import annotations

import torch

from ..nn.module import Parameter

ALIGN = 64


def _align(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


class FlatUnit:
    def __init__(self, name: str, params: list, world: int, rank: int, device, param_dtype):
        self.name = name
        self.params = params
        self.world, self.rank = world, rank
        self.device, self.dtype = device, param_dtype
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += _align(p.numel())
        self.numel = off
        self.padded = _align(max(off, 1), ALIGN * world)
        self.shard = self.padded // world
        lo = rank * self.shard

        # initial values -> fp32 master shard
        flat = torch.zeros(self.padded, dtype=torch.float32, device=device)
        for p, o in zip(params, self.offsets):
            flat[o:o + p.numel()].copy_(p.detach().reshape(-1).to(device=device, dtype=torch.float32))
        self.master = Parameter(flat[lo:lo + self.shard].clone(), requires_grad=True,
                                name=f"{name}.flat_shard")
        self.lp_shard = flat[lo:lo + self.shard].to(param_dtype)
        self._init_full = flat.to(param_dtype) if world == 1 else None
        del flat

        self.full = None          # low-precision full buffer the parameters view into
        self.grad_flat = None     # low-precision flat gradient (full size)
        self.grad_shard = None    # reduced gradient of this rank's shard
        self.pending = 0          # parameters whose gradient has not arrived yet in this backward
        self.grad_written = [False] * len(params)
        self.gather_event = None  # all-gather into `full` finished
        self.free_event = None    # last compute that read `full` finished
        self.reduce_event = None  # reduce-scatter of grad_flat finished
        self.gathered = False

    # ------------------------------------------------------------------ views
    def bind_full(self, buf: torch.Tensor) -> None:
        """Points every parameter at its slice of ``buf`` (done once; the addresses stay fixed)."""
        self.full = buf
        for p, o in zip(self.params, self.offsets):
            p.data = buf[o:o + p.numel()].view(p.shape)

    def bind_grad(self, buf: torch.Tensor) -> None:
        self.grad_flat = buf
        self.grad_views = [buf[o:o + p.numel()].view(p.shape) for p, o in zip(self.params, self.offsets)]

    def local_shard_of_full(self) -> torch.Tensor:
        lo = self.rank * self.shard
        return self.full[lo:lo + self.shard]

    def param_numel(self) -> int:
        return sum(p.numel() for p in self.params)
