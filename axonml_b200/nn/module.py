"""Module / Parameter / containers.

``Module`` is a ``torch.nn.Module`` that also answers the reference's trait methods
(crates/axonml-nn/src/module.rs:26-90): ``num_parameters``, ``set_training``, ``is_training``,
``name``; ``parameters()``/``named_parameters()``/``train``/``eval``/``zero_grad``/``forward``
come from torch with the same meaning.  ``Parameter`` mirrors parameter.rs:27-130 on top of
``torch.nn.Parameter``; ``Sequential``/``ModuleList`` mirror sequential.rs:35-140 and
module.rs:96-190 (children are named "0", "1", ... so state-dict keys are "<idx>.<param>").
"""
from __future__ import annotations

from typing import Iterable, Iterator

import torch


class Parameter(torch.nn.Parameter):
    """A trainable tensor with an optional name (parameter.rs:27-130)."""

    def __new__(cls, data=None, requires_grad: bool = True, name: str = ""):
        if data is None:
            data = torch.empty(0)
        obj = torch.Tensor._make_subclass(cls, torch.as_tensor(data), requires_grad)
        obj._axon_name = name
        return obj

    # constructors of the reference
    @classmethod
    def new(cls, data, requires_grad: bool = True) -> "Parameter":
        return cls(data, requires_grad)

    @classmethod
    def named(cls, name: str, data, requires_grad: bool = True) -> "Parameter":
        return cls(data, requires_grad, name)

    @classmethod
    def from_variable(cls, var) -> "Parameter":
        t = var.data if hasattr(var, "data") else var
        return cls(t, getattr(var, "requires_grad", True))

    def name(self) -> str:
        return getattr(self, "_axon_name", "")

    def set_name(self, name: str) -> None:
        self._axon_name = name

    def variable(self):
        return self

    def numel_(self) -> int:
        return self.numel()

    def zero_grad(self) -> None:
        self.grad = None

    def update_data(self, new_data: torch.Tensor) -> None:
        with torch.no_grad():
            self.copy_(new_data)

    def apply_update(self, update: torch.Tensor, lr: float = 1.0) -> None:
        with torch.no_grad():
            self.sub_(update, alpha=lr)

    def __reduce_ex__(self, proto):
        return (torch.nn.Parameter, (self.data, self.requires_grad))


class Module(torch.nn.Module):
    """Base class of every layer and model."""

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)

    def set_training(self, training: bool) -> "Module":
        return self.train(training)

    def is_training(self) -> bool:
        return self.training

    def name(self) -> str:
        return type(self).__name__

    def parameters_list(self) -> list:
        return list(self.parameters())

    def load_weights(self, weights: dict, prefix: str = "") -> int:
        """Copies ``weights[prefix + name]`` into every parameter and buffer of this module that
        has an entry (the per-layer ``load_weights`` of the reference's LLaMA blocks,
        crates/axonml-llm/src/llama.rs).  Returns how many tensors were loaded; a shape that does
        not match raises ``ValueError`` naming the tensor."""
        n = 0
        own = dict(self.named_parameters())
        own.update(dict(self.named_buffers()))
        with torch.no_grad():
            for name, dst in own.items():
                src = weights.get(prefix + name)
                if src is None:
                    continue
                src = torch.as_tensor(src)
                if src.shape != dst.shape:
                    raise ValueError(f"{prefix + name}: expected shape {tuple(dst.shape)}, got {tuple(src.shape)}")
                dst.copy_(src.to(dst.dtype))
                n += 1
        return n


class Sequential(torch.nn.Sequential, Module):
    """Ordered container; ``add``/``push`` append with automatic names "0", "1", ..."""

    @classmethod
    def new(cls) -> "Sequential":
        return cls()

    def add(self, module: torch.nn.Module) -> "Sequential":
        self.add_module(str(len(self)), module)
        return self

    def add_named(self, name: str, module: torch.nn.Module) -> "Sequential":
        self.add_module(name, module)
        return self

    def push(self, module: torch.nn.Module) -> None:
        self.add(module)

    def push_named(self, name: str, module: torch.nn.Module) -> None:
        self.add_named(name, module)

    def len(self) -> int:
        return len(self)

    def iter(self) -> Iterator[torch.nn.Module]:
        return iter(self)

    def is_empty(self) -> bool:
        return len(self) == 0


class ModuleList(torch.nn.ModuleList, Module):
    @classmethod
    def new(cls) -> "ModuleList":
        return cls()

    @classmethod
    def from_vec(cls, modules: Iterable[torch.nn.Module]) -> "ModuleList":
        return cls(list(modules))

    def push(self, module: torch.nn.Module) -> None:
        self.append(module)

    def get(self, index: int):
        return self[index] if -len(self) <= index < len(self) else None

    def len(self) -> int:
        return len(self)

    def iter_mut(self):
        """Modules are mutable objects here: the same iterator as ``iter``."""
        return iter(self)

    def iter(self):
        return iter(self)

    def is_empty(self) -> bool:
        return len(self) == 0
