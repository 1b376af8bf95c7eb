"""RMSprop (crates/axonml-optim/src/rmsprop.rs:84-250): ``sq = a*sq + (1-a)*g^2``; centered
subtracts the squared running mean of g; ``avg = sqrt(.) + eps``; optional momentum buffer."""
from __future__ import annotations

import torch

from ..ops import optim as O
from .optimizer import Optimizer


class RMSprop(Optimizer):
    def __init__(self, params, lr: float = 1e-2, alpha: float = 0.99, eps: float = 1e-8,
                 weight_decay: float = 0.0, momentum: float = 0.0, centered: bool = False):
        super().__init__(params, lr)
        self._alpha, self._eps, self._weight_decay = alpha, eps, weight_decay
        self._momentum, self._centered = momentum, centered

    @classmethod
    def new(cls, params, lr): return cls(params, lr)

    @classmethod
    def with_alpha(cls, params, lr, alpha): return cls(params, lr, alpha)

    @classmethod
    def with_options(cls, params, lr, alpha, eps, weight_decay, momentum, centered):
        return cls(params, lr, alpha, eps, weight_decay, momentum, centered)

    def alpha(self, a): self._alpha = a; return self
    def eps(self, e): self._eps = e; return self
    def weight_decay(self, wd): self._weight_decay = wd; return self
    def momentum(self, m): self._momentum = m; return self
    def centered(self, flag=True): self._centered = flag; return self

    def _hyper(self):
        return {"_alpha": self._alpha, "_eps": self._eps, "_weight_decay": self._weight_decay,
                "_momentum": self._momentum, "_centered": self._centered}

    @torch.no_grad()
    def step(self) -> None:
        names = ("square_avg", "momentum_buffer", "grad_avg")
        fused, rest = self._groups(self._active())
        for grp in fused:
            sts = [self._state(p, names) for p in grp]
            O.multi_tensor("rmsprop", grp, [self._g(p) for p in grp], [s["square_avg"] for s in sts],
                           [s["momentum_buffer"] for s in sts], [s["grad_avg"] for s in sts],
                           lp=self._lp(grp), lr=self.lr, alpha=self._alpha, eps=self._eps, wd=self._weight_decay,
                           momentum=self._momentum, centered=self._centered,
                           inv_scale=self._inv_scale, found_inf=self._found_inf)
        if rest and not self._skip():
            for p in rest:
                st = self._state(p, names)
                g = self._grad(p)
                pf = p.float()
                if self._weight_decay:
                    g = g + self._weight_decay * pf
                sq = st["square_avg"]
                sq.mul_(self._alpha).addcmul_(g, g, value=1 - self._alpha)
                if self._centered:
                    ga = st["grad_avg"]
                    ga.mul_(self._alpha).add_(g, alpha=1 - self._alpha)
                    avg = (sq - ga * ga).clamp_min(0).sqrt() + self._eps
                else:
                    avg = sq.sqrt() + self._eps
                if self._momentum > 0:
                    buf = st["momentum_buffer"]
                    buf.mul_(self._momentum).add_(g / avg)
                    pf = pf - self.lr * buf
                else:
                    pf = pf - self.lr * g / avg
                self._write(p, pf.to(p.dtype))
        self._step_count += 1
