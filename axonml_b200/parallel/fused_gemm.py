"""Sequence-parallel linear layers: all-gather -> GEMM and GEMM -> reduce-scatter.

``all_gather_linear(x_local, W, ...)``: ``x_local`` holds this rank's tokens ``[T/world, K]``; the
result is ``act([x_0; x_1; ...] W^T + b)`` for all ``T`` tokens.
``linear_reduce_scatter(x, W)``: every rank holds a partial product over its slice of the reduction
dim; the result is this rank's ``T/world`` tokens of the summed output.

On a B200 box with symmetric memory these run as ONE kernel each (``csrc/kernels/gemm_comm.cu``):
the GEMM's tile order follows the arrival of the peers' shards, respectively pushes finished
tiles to their owner over NVLink while later tiles are still being computed.  Elsewhere (CPU
ranks, a single rank, unsupported shapes) the same result is composed from the process group's
collectives, which is also the baseline the fused kernels are measured against.
"""
from __future__ import annotations

import torch

from ..ops.linear import linear
from . import tensor_parallel as TP

_ENGINES: dict = {}


def _engine(pg):
    """Per-process-group fused engine, or None when the fused path cannot be used."""
    key = id(pg.backend())
    if key not in _ENGINES:
        eng = None
        try:
            from . import gemm_comm
            eng = gemm_comm.FusedGemmComm.try_create(pg)
        except Exception:
            eng = None
        _ENGINES[key] = eng
    return _ENGINES[key]


def all_gather_linear(x_local, weight, bias=None, act: str = "none", pg=None):
    lead = x_local.shape[:-1]
    x2 = x_local.reshape(-1, x_local.shape[-1])
    eng = _engine(pg) if pg.world_size() > 1 else None
    if eng is not None and eng.supports_ag(x2, weight):
        y = eng.all_gather_linear(x2, weight, bias, act)
    else:
        y = linear(TP.all_gather_tokens(x2, pg), weight, bias, act)
    if len(lead) > 1:
        return y.view(lead[0] * pg.world_size(), *lead[1:], y.shape[-1])
    return y


def linear_reduce_scatter(x, weight, pg=None):
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    eng = _engine(pg) if pg.world_size() > 1 else None
    if eng is not None and eng.supports_rs(x2, weight):
        y = eng.linear_reduce_scatter(x2, weight)
    else:
        y = TP.reduce_scatter_tokens(linear(x2, weight), pg)
    if len(lead) > 1:
        return y.view(lead[0] // pg.world_size(), *lead[1:], y.shape[-1])
    return y
