"""StateDict containers (crates/axonml-serialize/src/state_dict.rs:16-260): ``TensorData``,
``StateDictEntry``, ``StateDict`` with ``from_module / insert / get / merge / filter_prefix /
strip_prefix / add_prefix / summary``.  ``from_module`` uses fully-qualified names and includes
buffers (the reference uses bare "weight"/"bias" names that collide across layers and drops
BatchNorm running statistics)."""
from __future__ import annotations

import dataclasses

import torch


@dataclasses.dataclass
class TensorData:
    shape: list
    values: torch.Tensor          # flat fp32

    @classmethod
    def from_tensor(cls, t: torch.Tensor) -> "TensorData":
        return cls(list(t.shape), t.detach().to("cpu", torch.float32).reshape(-1).contiguous())

    def to_tensor(self) -> torch.Tensor:
        return self.values.view(self.shape)

    def numel(self) -> int:
        return self.values.numel()


@dataclasses.dataclass
class StateDictEntry:
    data: TensorData
    requires_grad: bool = True
    metadata: dict = dataclasses.field(default_factory=dict)

    @classmethod
    def new(cls, data: TensorData, requires_grad: bool = True): return cls(data, requires_grad)

    def with_metadata(self, key: str, value: str) -> "StateDictEntry":
        self.metadata[key] = value
        return self


class StateDict:
    def __init__(self):
        self._entries: dict[str, StateDictEntry] = {}
        self.metadata: dict[str, str] = {}

    @classmethod
    def new(cls): return cls()

    @classmethod
    def from_module(cls, module: torch.nn.Module) -> "StateDict":
        sd = cls()
        for name, p in module.named_parameters():
            sd.insert_entry(name, StateDictEntry(TensorData.from_tensor(p), p.requires_grad))
        for name, b in module.named_buffers():
            sd.insert_entry(name, StateDictEntry(TensorData.from_tensor(b.float()), False, {"buffer": "true"}))
        return sd

    @classmethod
    def from_tensors(cls, tensors: dict) -> "StateDict":
        sd = cls()
        for k, v in tensors.items():
            sd.insert(k, TensorData.from_tensor(torch.as_tensor(v)))
        return sd

    def insert(self, name: str, data: TensorData) -> None:
        self._entries[name] = StateDictEntry(data, True)

    def insert_entry(self, name: str, entry: StateDictEntry) -> None:
        self._entries[name] = entry

    def get(self, name: str): return self._entries.get(name)
    def get_mut(self, name: str): return self._entries.get(name)
    def contains(self, name: str) -> bool: return name in self._entries
    def __contains__(self, name: str) -> bool: return name in self._entries
    def __len__(self) -> int: return len(self._entries)
    def len(self) -> int: return len(self._entries)
    def is_empty(self) -> bool: return not self._entries
    def keys(self): return self._entries.keys()
    def entries(self): return self._entries.items()
    def remove(self, name: str): return self._entries.pop(name, None)

    def merge(self, other: "StateDict") -> None:
        self._entries.update(other._entries)
        self.metadata.update(other.metadata)

    def filter_prefix(self, prefix: str) -> "StateDict":
        out = StateDict()
        out._entries = {k: v for k, v in self._entries.items() if k.startswith(prefix)}
        return out

    def strip_prefix(self, prefix: str) -> "StateDict":
        out = StateDict()
        out._entries = {(k[len(prefix):] if k.startswith(prefix) else k): v for k, v in self._entries.items()}
        out.metadata = dict(self.metadata)
        return out

    def add_prefix(self, prefix: str) -> "StateDict":
        out = StateDict()
        out._entries = {prefix + k: v for k, v in self._entries.items()}
        out.metadata = dict(self.metadata)
        return out

    def set_metadata(self, key: str, value: str) -> None: self.metadata[key] = value
    def get_metadata(self, key: str): return self.metadata.get(key)
    def total_params(self) -> int: return sum(e.data.numel() for e in self._entries.values())
    def size_bytes(self) -> int: return 4 * self.total_params()

    def summary(self) -> str:
        lines = [f"StateDict: {len(self)} tensors, {self.total_params()} parameters, {self.size_bytes()} bytes"]
        for k, e in self._entries.items():
            lines.append(f"  {k}: {e.data.shape}")
        return "\n".join(lines)

    def to_tensors(self) -> dict:
        return {k: e.data.to_tensor() for k, e in self._entries.items()}

    def load_into(self, module: torch.nn.Module, strict: bool = True) -> list:
        """Copies matching entries into ``module`` (parameters and buffers).  Files written by the
        reference carry unqualified names; an entry is also accepted when exactly one module
        tensor ends with ``.<key>`` or equals it and the shapes agree.  Returns the list of module
        tensors that found no entry."""
        own = dict(module.named_parameters())
        own.update(dict(module.named_buffers()))
        missing = []
        with torch.no_grad():
            for name, t in own.items():
                e = self._entries.get(name)
                if e is None:
                    short = name.rsplit(".", 1)[-1]
                    cands = [k for k in own if k.rsplit(".", 1)[-1] == short]
                    if len(cands) == 1 and short in self._entries:
                        e = self._entries[short]
                if e is None or list(e.data.shape) != list(t.shape):
                    missing.append(name)
                    continue
                t.copy_(e.data.to_tensor().to(t.dtype))
        if strict and missing:
            raise KeyError(f"state dict is missing {missing}")
        return missing
