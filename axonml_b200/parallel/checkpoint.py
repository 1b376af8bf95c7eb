"""Sharded training checkpoints for the fully-sharded engine, resumable at another world size.

Every rank writes one file, ``shard_{rank:05d}.axonml`` (the bincode StateDict container of
``serialize``: fp32 tensors keyed ``{unit}.master``, ``{unit}.exp_avg``, ``{unit}.exp_avg_sq``),
rank 0 also writes ``manifest.json``: world size, optimizer step, per-unit logical length and the
parameter layout (name, offset, shape) inside each unit's flat range.  A flat unit is a 1-D array
split evenly over the ranks, so loading at a different world size is pure index arithmetic: the new
rank's range ``[r*S', (r+1)*S')`` is cut from the old shard files that overlap it.  Nothing is
gathered on one GPU or one host.

The reference documents a ``CheckpointManager`` but ships none (Axonml_Architecture.md:438-473);
its ``Checkpoint`` container (crates/axonml-serialize/src/checkpoint.rs:121-137) holds an unsharded
model only.
"""
from __future__ import annotations

import json
import os

import torch

from ..serialize import load_state_dict, save_state_dict
from ..serialize.state_dict import StateDict

_KEYS = ("master", "exp_avg", "exp_avg_sq")


def _unit_moments(engine, optimizer, u):
    """fp32 moment shards of a unit: the fused in-backward AdamW keeps them on the unit, a separate
    optimizer keeps them in its per-parameter state."""
    if getattr(u, "m1", None) is not None:
        return u.m1, u.m2
    st = getattr(optimizer, "state", {}).get(id(u.master)) if optimizer is not None else None
    if st and "exp_avg" in st:
        return st["exp_avg"], st["exp_avg_sq"]
    return None, None


def save_sharded(directory: str, engine, optimizer=None, step: int = 0, extra: dict | None = None) -> None:
    os.makedirs(directory, exist_ok=True)
    rank, world = engine.rank, engine.world
    tensors = {}
    for u in engine.units:
        tensors[f"{u.name}.master"] = u.master.detach().float().cpu()
        m1, m2 = _unit_moments(engine, optimizer, u)
        if m1 is not None:
            tensors[f"{u.name}.exp_avg"] = m1.detach().float().cpu()
            tensors[f"{u.name}.exp_avg_sq"] = m2.detach().float().cpu()
    if all(u.world == 1 for u in engine.units) and rank != 0:
        tensors = {}                      # replicated (NoShard): rank 0's file is the whole state
    save_state_dict(StateDict.from_tensors(tensors), os.path.join(directory, f"shard_{rank:05d}.axonml"))
    if rank == 0:
        names = {id(p): n for n, p in engine.module.named_parameters()}
        manifest = {
            "format": "axonml-sharded-v1", "world_size": world, "step": int(step),
            "optimizer_step": int(getattr(optimizer, "_step_count", getattr(engine, "_fused_step", 0)) or 0),
            "units": [{"name": u.name, "numel": u.numel, "padded": u.padded, "shard": u.shard, "sharded": u.world > 1,
                       "params": [{"name": names[id(p)], "offset": o, "shape": list(p.shape)}
                                  for p, o in zip(u.params, u.offsets)]} for u in engine.units],
            "extra": extra or {},
        }
        with open(os.path.join(directory, "manifest.json"), "w") as f:
            json.dump(manifest, f, indent=1)
    engine.pg.barrier()


class _ShardReader:
    """Lazily opened shard files of a saved run."""

    def __init__(self, directory: str):
        self.dir, self._open = directory, {}

    def get(self, rank: int, key: str):
        if rank not in self._open:
            self._open[rank] = load_state_dict(os.path.join(self.dir, f"shard_{rank:05d}.axonml")).to_tensors()
        return self._open[rank].get(key)


def _cut(reader: _ShardReader, unit: dict, key: str, lo: int, hi: int, old_world: int):
    """Elements ``[lo, hi)`` of a unit's logical flat array from the old shard files (zeros past the
    old padded length).  Returns None when the key was not saved."""
    out = torch.zeros(hi - lo, dtype=torch.float32)
    if not unit["sharded"]:
        src = reader.get(0, key)
        if src is None:
            return None
        n = max(0, min(hi, src.numel()) - lo)
        if n > 0:
            out[:n] = src[lo:lo + n]
        return out
    s_old = unit["shard"]
    found = False
    for r in range(lo // s_old, min(old_world, (hi + s_old - 1) // s_old)):
        src = reader.get(r, key)
        if src is None:
            continue
        found = True
        a, b = max(lo, r * s_old), min(hi, (r + 1) * s_old)
        if b > a:
            out[a - lo:b - lo] = src[a - r * s_old:b - r * s_old]
    return out if found else None


def load_sharded(directory: str, engine, optimizer=None) -> dict:
    """Restores master weights, low-precision shards and Adam moments into ``engine`` (built for the
    current world size, same model and unit partition).  Returns the manifest."""
    with open(os.path.join(directory, "manifest.json")) as f:
        manifest = json.load(f)
    if manifest.get("format") != "axonml-sharded-v1":
        raise ValueError("not a sharded axonml checkpoint")
    old_world = manifest["world_size"]
    by_name = {u["name"]: u for u in manifest["units"]}
    reader = _ShardReader(directory)
    for u in engine.units:
        mu = by_name.get(u.name)
        if mu is None or mu["numel"] != u.numel:
            raise ValueError(f"unit {u.name} does not match the checkpoint (model or unit partition differs)")
        lo = u.rank * u.shard if u.world > 1 else 0
        hi = lo + u.shard
        new = {k: _cut(reader, mu, f"{u.name}.{k}", lo, hi, old_world) for k in _KEYS}
        with torch.no_grad():
            u.master.copy_(new["master"].to(u.master.device))
            u.lp_shard.copy_(u.master.to(u.lp_shard.dtype))
            if u.world > 1:
                u.gathered = False
            m1, m2 = _unit_moments(engine, optimizer, u)
            if new["exp_avg"] is not None:
                if m1 is None and optimizer is not None and hasattr(optimizer, "_state"):
                    st = optimizer._state(u.master, ("exp_avg", "exp_avg_sq"))
                    m1, m2 = st["exp_avg"], st["exp_avg_sq"]
                if m1 is not None:
                    m1.copy_(new["exp_avg"].to(m1.device))
                    m2.copy_(new["exp_avg_sq"].to(m2.device))
    step = manifest.get("optimizer_step", 0)
    if optimizer is not None and hasattr(optimizer, "_step_count"):
        optimizer._step_count = step
    if hasattr(engine, "_fused_step") and getattr(engine, "_fused", None) is not None:
        engine._fused_step = step
    engine.pg.barrier()
    return manifest
