"""Optimizer base class.  Reference trait: crates/axonml-optim/src/optimizer.rs:17-39
(``step, zero_grad, get_lr, set_lr, parameters, num_parameters``).  Unlike the reference the
optimizers carry a ``state_dict`` so that checkpoints restore momentum / Adam moments.

On CUDA every step is a multi-tensor fused kernel (``ops.optim``): parameters are grouped by
(param dtype, grad dtype) and updated in a handful of launches, with the GradScaler's 1/scale and
found-inf flag read from device memory.  On CPU the same formulas run as torch expressions."""
from __future__ import annotations

from typing import Iterable

import torch

from ..ops import optim as O


class ParamState:
    """Per-parameter optimizer state (optimizer.rs:49-84): ``momentum_buffer`` (SGD momentum, or
    Adam's first moment), ``exp_avg_sq`` (second moment), ``max_exp_avg_sq`` (AMSGrad) and the
    ``step`` count.  ``Optimizer.param_state(p)`` returns the live state of a parameter in this
    form; the buffers are the fp32 tensors the update kernels work on, not copies."""

    def __init__(self, momentum_buffer=None, exp_avg_sq=None, max_exp_avg_sq=None, step: int = 0):
        self.momentum_buffer, self.exp_avg_sq, self.max_exp_avg_sq, self.step = momentum_buffer, exp_avg_sq, max_exp_avg_sq, step

    @classmethod
    def new(cls): return cls()

    def init_momentum(self, size, device=None) -> None:
        self.momentum_buffer = torch.zeros(size, dtype=torch.float32, device=device)

    def init_exp_avg_sq(self, size, device=None) -> None:
        self.exp_avg_sq = torch.zeros(size, dtype=torch.float32, device=device)

    def __repr__(self) -> str:
        has = [n for n in ("momentum_buffer", "exp_avg_sq", "max_exp_avg_sq") if getattr(self, n) is not None]
        return f"ParamState(step={self.step}, buffers={has})"


# names under which the optimizers keep the buffers of a ParamState
_FIRST_MOMENT = ("momentum_buffer", "buf", "exp_avg", "m", "grad_avg")
_SECOND_MOMENT = ("exp_avg_sq", "v", "square_avg", "sq")
_MAX_SECOND = ("max_exp_avg_sq", "vmax", "max_v")


class Optimizer:
    def __init__(self, params: Iterable[torch.Tensor], lr: float):
        self.params = [p for p in params]
        if not self.params:
            raise ValueError("optimizer got an empty parameter list")
        self.lr = float(lr)
        self.state: dict[int, dict] = {}
        self._step_count = 0
        # set by GradScaler.step(): device tensors read by the fused kernels
        self._inv_scale = None
        self._found_inf = None

    # ---- reference trait
    def step(self) -> None:  # pragma: no cover - abstract
        raise NotImplementedError

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if getattr(p, "_axon_grad", None) is not None:
                p._axon_grad = None
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    def get_lr(self) -> float:
        return self.lr

    def set_lr(self, lr: float) -> None:
        self.lr = float(lr)

    def parameters(self):
        return self.params

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.params)

    def param_state(self, p) -> ParamState:
        """The state kept for parameter ``p`` as a ``ParamState`` (empty before the first step)."""
        st = self.state.get(id(p), {})
        pick = lambda names: next((st[n] for n in names if n in st), None)
        return ParamState(pick(_FIRST_MOMENT), pick(_SECOND_MOMENT), pick(_MAX_SECOND), self._step_count)

    # torch-style view used by the schedulers
    @property
    def param_groups(self):
        return [{"params": self.params, "lr": self.lr}]

    # ---- helpers
    def _state(self, p, names):
        st = self.state.get(id(p))
        if st is None:
            st = {n: torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
                  for n in names}
            self.state[id(p)] = st
        else:
            for n in names:
                if n not in st:
                    st[n] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
        return st

    @staticmethod
    def _g(p):
        """Gradient of ``p``: a sharded engine may attach it as ``_axon_grad`` (it can have a
        different dtype than the master parameter, which ``.grad`` does not allow)."""
        g = getattr(p, "_axon_grad", None)
        return g if g is not None else p.grad

    @staticmethod
    def _lp(grp):
        """Low-precision mirrors the kernel refreshes together with the fp32 parameters."""
        lps = [getattr(p, "_axon_lp", None) for p in grp]
        return lps if any(l is not None for l in lps) else None

    @staticmethod
    def _write(p, new) -> None:
        p.copy_(new)
        lp = getattr(p, "_axon_lp", None)
        if lp is not None:
            lp.copy_(p)

    def _active(self):
        return [p for p in self.params if self._g(p) is not None]

    def _device_step(self, device):
        """Steps actually taken, as an int32 device scalar, for the kernels' bias corrections while
        a device-side found-inf flag may skip steps (the host counter would run ahead after every
        overflow).  None when no such flag is attached."""
        if self._found_inf is None or not torch.is_tensor(self._found_inf) or not self._found_inf.is_cuda:
            return None
        st = getattr(self, "_step_dev", None)
        if st is None or st.device != device:
            # the host count includes the step in progress
            st = self._step_dev = torch.full((1,), max(self._step_count - 1, 0), dtype=torch.int32, device=device)
        return st

    def _advance_device_step(self) -> None:
        st = getattr(self, "_step_dev", None)
        if st is not None and self._found_inf is not None and torch.is_tensor(self._found_inf):
            st += (self._found_inf.to(st.device) == 0).to(torch.int32)

    def _groups(self, ps):
        """Splits into lists the fused kernel can take plus a remainder for the torch path."""
        fused: dict[tuple, list] = {}
        rest = []
        for p in ps:
            g = self._g(p)
            if (p.is_cuda and O.supported([p], [g]) and not g.is_sparse):
                fused.setdefault((p.dtype, g.dtype, p.device, getattr(p, '_axon_lp', None) is not None), []).append(p)
            else:
                rest.append(p)
        return list(fused.values()), rest

    def _skip(self) -> bool:
        """CPU-side found-inf check for the torch path."""
        return self._found_inf is not None and bool(self._found_inf.item())

    def _grad(self, p):
        g = self._g(p).float()
        if self._inv_scale is not None:
            g = g * self._inv_scale.to(g.device)
        return g

    # ---- state dict
    def state_dict(self) -> dict:
        out = {"lr": self.lr, "step": self._step_count, "state": {}, "hyper": self._hyper()}
        for i, p in enumerate(self.params):
            st = self.state.get(id(p))
            if st:
                out["state"][i] = {k: v.detach().clone() if torch.is_tensor(v) else v for k, v in st.items()}
        return out

    def load_state_dict(self, sd: dict) -> None:
        self.lr = float(sd.get("lr", self.lr))
        self._step_count = int(sd.get("step", 0))
        for i, st in sd.get("state", {}).items():
            p = self.params[int(i)]
            self.state[id(p)] = {k: (v.to(p.device) if torch.is_tensor(v) else v) for k, v in st.items()}
        for k, v in sd.get("hyper", {}).items():
            if hasattr(self, k):
                setattr(self, k, v)

    def _hyper(self) -> dict:
        return {}
