"""Model inference service (crates/axonml-server/src/inference/server.rs:263-423, pool.rs:82-125):
``InferenceServer`` builds a ``Sequential`` from a StateDict once per model (the reference rebuilds
it for every request), ``ModelPool`` keeps up to 100 loaded models and evicts entries idle for more
than 300 s."""
from __future__ import annotations

import threading
import time

import torch

from .. import nn
from ..serialize import StateDict, load_state_dict


def build_model_from_state_dict(sd: StateDict, activation: str = "relu") -> nn.Sequential:
    """MLP from ``<i>.weight`` / ``<i>.bias`` (or ``fc<i>`` / ``layers.<i>``) entries, ordered by index."""
    layers = {}
    for k, e in sd.entries():
        if k.endswith(".weight") and len(e.data.shape) == 2:
            stem = k[:-7]
            digits = "".join(c for c in stem if c.isdigit())
            layers[stem] = (int(digits) if digits else len(layers), e.data.to_tensor())
    model = nn.Sequential()
    ordered = sorted(layers.items(), key=lambda kv: kv[1][0])
    for i, (stem, (_, w)) in enumerate(ordered):
        b = sd.get(stem + ".bias")
        model.add(nn.Linear.from_weights(w, b.data.to_tensor() if b is not None else None))
        if i + 1 < len(ordered):
            model.add({"relu": nn.ReLU, "tanh": nn.Tanh, "sigmoid": nn.Sigmoid, "gelu": nn.GELU}[activation]())
    return model.eval()


class ModelPool:
    def __init__(self, max_entries: int = 100, idle_timeout_s: float = 300.0):
        self.max_entries, self.idle = max_entries, idle_timeout_s
        self._d: dict = {}
        self._lock = threading.Lock()

    def acquire(self, name: str, loader):
        with self._lock:
            self.evict_idle()
            ent = self._d.get(name)
            if ent is None:
                if len(self._d) >= self.max_entries:
                    oldest = min(self._d, key=lambda k: self._d[k][1])
                    del self._d[oldest]
                ent = [loader(), time.time(), 0]
                self._d[name] = ent
            ent[1] = time.time()
            ent[2] += 1
            return ent[0]

    def release(self, name: str) -> None:
        with self._lock:
            if name in self._d:
                self._d[name][2] = max(0, self._d[name][2] - 1)

    def evict_idle(self) -> int:
        now = time.time()
        dead = [k for k, (m, t, users) in self._d.items() if users == 0 and now - t > self.idle]
        for k in dead:
            del self._d[k]
        return len(dead)

    def len(self) -> int: return len(self._d)
    def contains(self, name: str) -> bool: return name in self._d


class InferenceServer:
    def __init__(self, device=None):
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.models: dict = {}
        self.pool = ModelPool()

    @classmethod
    def new(cls): return cls()

    def register(self, name: str, model) -> None:
        self.models[name] = model.to(self.device).eval()

    def load(self, name: str, path: str, activation: str = "relu") -> None:
        self.register(name, build_model_from_state_dict(load_state_dict(path), activation))

    def unload(self, name: str) -> None: self.models.pop(name, None)
    def list_models(self): return sorted(self.models)

    @torch.no_grad()
    def predict(self, name: str, inputs) -> list:
        if name not in self.models:
            raise KeyError(f"unknown model {name}")
        x = torch.as_tensor(inputs, dtype=torch.float32, device=self.device)
        single = x.dim() == 1
        y = self.models[name](x.unsqueeze(0) if single else x)
        return (y[0] if single else y).float().cpu().tolist()
