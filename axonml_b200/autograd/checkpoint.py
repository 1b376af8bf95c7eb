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


def estimate_memory_savings(num_layers: int, segments: int, activation_size_mb: float) -> tuple:
    """(MB of activations kept without checkpointing, MB kept with ``segments`` segments): without,
    every layer's activation is held; with, ``ceil(num_layers / segments)`` are (checkpoint.rs:175-187)."""
    without = num_layers * activation_size_mb
    if segments <= 0:
        return without, without
    return without, -(-num_layers // segments) * activation_size_mb


def suggest_segments(num_layers: int, activation_size_mb: float, available_memory_mb: float) -> int:
    """Segments to split a stack into so that the stored activations fit: 0 when everything fits,
    ``num_layers`` when not even one activation does, else ``ceil(num_layers / storable)``
    (checkpoint.rs:199-221)."""
    if num_layers * activation_size_mb <= available_memory_mb:
        return 0
    storable = int(available_memory_mb // activation_size_mb) if activation_size_mb > 0 else num_layers
    if storable == 0:
        return num_layers
    return -(-num_layers // storable)
