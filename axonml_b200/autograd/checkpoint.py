"""Activation checkpointing with real recomputation
(API of crates/axonml-autograd/src/checkpoint.rs:70,120)."""
from __future__ import annotations

import torch
import torch.utils.checkpoint as _ckpt


def checkpoint(function, *inputs, **kwargs):
    """Runs ``function(*inputs)`` without storing its intermediates; they are recomputed during
    backward."""
    if not torch.is_grad_enabled():
        return function(*inputs, **kwargs)
    return _ckpt.checkpoint(function, *inputs, use_reentrant=False, **kwargs)


def checkpoint_sequential(num_layers: int, segments: int, input, layer_fn):
    """Splits ``num_layers`` layers into ``segments`` checkpointed groups; ``layer_fn(i, x)``
    applies layer i."""
    segments = max(1, min(segments, num_layers))
    per = (num_layers + segments - 1) // segments
    x = input
    for s in range(0, num_layers, per):
        def run(x, s=s):
            for i in range(s, min(s + per, num_layers)):
                x = layer_fn(i, x)
            return x
        x = checkpoint(run, x)
    return x
