"""Free-function collectives (crates/axonml-distributed/src/comm.rs:17-203)."""
from __future__ import annotations

import torch

from .backend import ReduceOp
from .process_group import ProcessGroup


def all_reduce_sum(t, pg: ProcessGroup): return pg.all_reduce_tensor(t, ReduceOp.Sum)
def all_reduce_mean(t, pg: ProcessGroup): return pg.all_reduce_tensor(t, ReduceOp.Average)
def all_reduce_min(t, pg: ProcessGroup): return pg.all_reduce_tensor(t, ReduceOp.Min)
def all_reduce_max(t, pg: ProcessGroup): return pg.all_reduce_tensor(t, ReduceOp.Max)
def all_reduce_product(t, pg: ProcessGroup): return pg.all_reduce_tensor(t, ReduceOp.Product)
def broadcast(t, pg: ProcessGroup): return pg.broadcast_tensor(t, 0)
def broadcast_from(t, src: int, pg: ProcessGroup): return pg.broadcast_tensor(t, src)
def all_gather(t, pg: ProcessGroup): return pg.all_gather_tensor(t)
def reduce_scatter_sum(t, pg: ProcessGroup): return pg.reduce_scatter_tensor(t, ReduceOp.Sum)
def reduce_scatter_mean(t, pg: ProcessGroup): return pg.reduce_scatter_tensor(t, ReduceOp.Average)
def barrier(pg: ProcessGroup): pg.barrier()
def is_main_process(pg: ProcessGroup) -> bool: return pg.rank() == 0
def world_size(pg: ProcessGroup) -> int: return pg.world_size()
def rank(pg: ProcessGroup) -> int: return pg.rank()


def scatter_tensor(t: torch.Tensor, pg: ProcessGroup) -> torch.Tensor:
    """This rank's dim-0 slice of ``t`` (comm.rs:114-140)."""
    w, r = pg.world_size(), pg.rank()
    n = t.shape[0] // w
    return t[r * n:(r + 1) * n].clone()


def gather_tensor(t: torch.Tensor, pg: ProcessGroup) -> torch.Tensor:
    """Concatenation along dim 0 of every rank's ``t`` (comm.rs:142-171)."""
    g = pg.all_gather_tensor(t)
    return g.reshape((-1,) + tuple(t.shape[1:]))


def sync_gradient(grad: torch.Tensor, pg: ProcessGroup) -> torch.Tensor:
    return pg.all_reduce_tensor(grad, ReduceOp.Average)


def sync_gradients(grads, pg: ProcessGroup):
    for g in grads:
        sync_gradient(g, pg)
    return grads


def ring_all_reduce(t: torch.Tensor, pg: ProcessGroup, op: ReduceOp = ReduceOp.Sum) -> torch.Tensor:
    return pg.all_reduce_tensor(t, op)
