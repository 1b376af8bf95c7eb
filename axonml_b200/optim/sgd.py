"""SGD (crates/axonml-optim/src/sgd.rs:52-198): ``g += wd*p``; the first step copies the
gradient into the momentum buffer, later steps ``buf = m*buf + (1-dampening)*g``; nesterov uses
``g + m*buf``; ``p -= lr*g``."""
from __future__ import annotations

import torch

from ..ops import optim as O
from .optimizer import Optimizer


class SGD(Optimizer):
    def __init__(self, params, lr: float, momentum: float = 0.0, weight_decay: float = 0.0,
                 dampening: float = 0.0, nesterov: bool = False):
        super().__init__(params, lr)
        self._momentum, self._weight_decay = momentum, weight_decay
        self._dampening, self._nesterov = dampening, nesterov

    @classmethod
    def new(cls, params, lr): return cls(params, lr)

    @classmethod
    def with_momentum(cls, params, lr, momentum): return cls(params, lr, momentum)

    @classmethod
    def with_options(cls, params, lr, momentum, weight_decay, dampening, nesterov):
        return cls(params, lr, momentum, weight_decay, dampening, nesterov)

    # chainable builders
    def momentum(self, m): self._momentum = m; return self
    def weight_decay(self, wd): self._weight_decay = wd; return self
    def nesterov(self, flag=True): self._nesterov = flag; return self
    def dampening(self, d): self._dampening = d; return self

    def _hyper(self):
        return {"_momentum": self._momentum, "_weight_decay": self._weight_decay,
                "_dampening": self._dampening, "_nesterov": self._nesterov}

    @torch.no_grad()
    def step(self) -> None:
        ps = self._active()
        fused, rest = self._groups(ps)
        for grp in fused:
            if self._momentum == 0.0:
                subsets = [(grp, True)]
            else:
                fresh = [p for p in grp if not self.state.get(id(p), {}).get("_init")]
                seen = [p for p in grp if self.state.get(id(p), {}).get("_init")]
                subsets = [(fresh, True), (seen, False)]
            for sub, first in subsets:
                if not sub:
                    continue
                bufs = None
                if self._momentum != 0.0:
                    bufs = [self._state(p, ("momentum_buffer",))["momentum_buffer"] for p in sub]
                O.multi_tensor("sgd", sub, [self._g(p) for p in sub], bufs, lp=self._lp(sub), lr=self.lr,
                               momentum=self._momentum, wd=self._weight_decay,
                               dampening=self._dampening, nesterov=self._nesterov,
                               first_step=first, inv_scale=self._inv_scale,
                               found_inf=self._found_inf)
                if self._momentum != 0.0:
                    for p in sub:
                        self.state[id(p)]["_init"] = True
        if rest and not self._skip():
            for p in rest:
                g = self._grad(p)
                pf = p.float()
                if self._weight_decay:
                    g = g + self._weight_decay * pf
                if self._momentum != 0.0:
                    new = id(p) not in self.state or not self.state[id(p)].get("_init")
                    st = self._state(p, ("momentum_buffer",))
                    buf = st["momentum_buffer"]
                    if new:
                        buf.copy_(g)
                        st["_init"] = True
                    else:
                        buf.mul_(self._momentum).add_(g, alpha=1 - self._dampening)
                    g = g + self._momentum * buf if self._nesterov else buf
                self._write(p, (pf - self.lr * g).to(p.dtype))
        self._step_count += 1
