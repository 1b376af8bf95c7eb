"""Adam / AdamW (crates/axonml-optim/src/adam.rs:76-445).  Adam adds L2 weight decay into the
gradient; AdamW decays the parameter directly (``p *= 1 - lr*wd``, default wd 0.01).  Step size
``lr / (1-beta1^t)``, denominator ``sqrt(v / (1-beta2^t)) + eps``; optional amsgrad."""
from __future__ import annotations

import torch

from ..ops import optim as O
from .optimizer import Optimizer


class Adam(Optimizer):
    _DECOUPLED = False
    _DEFAULT_WD = 0.0

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float | None = None, amsgrad: bool = False):
        super().__init__(params, lr)
        self._betas = tuple(betas)
        self._eps = eps
        self._weight_decay = self._DEFAULT_WD if weight_decay is None else weight_decay
        self._amsgrad = amsgrad

    @classmethod
    def new(cls, params, lr): return cls(params, lr)

    @classmethod
    def with_betas(cls, params, lr, betas): return cls(params, lr, betas)

    @classmethod
    def with_options(cls, params, lr, betas, eps, weight_decay, amsgrad=False):
        return cls(params, lr, betas, eps, weight_decay, amsgrad)

    def betas(self, b1, b2=None):
        self._betas = tuple(b1) if b2 is None else (b1, b2)
        return self

    def eps(self, e): self._eps = e; return self
    def weight_decay(self, wd): self._weight_decay = wd; return self
    def amsgrad(self, flag=True): self._amsgrad = flag; return self

    def _hyper(self):
        return {"_betas": self._betas, "_eps": self._eps, "_weight_decay": self._weight_decay,
                "_amsgrad": self._amsgrad}

    @torch.no_grad()
    def step(self) -> None:
        self._step_count += 1
        t = self._step_count
        b1, b2 = self._betas
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
        names = ("exp_avg", "exp_avg_sq") + (("max_exp_avg_sq",) if self._amsgrad else ())
        fused, rest = self._groups(self._active())
        step_dev = self._device_step(fused[0][0].device) if fused else None
        for grp in fused:
            sts = [self._state(p, names) for p in grp]
            O.multi_tensor("adam", grp, [self._g(p) for p in grp], [s["exp_avg"] for s in sts],
                           [s["exp_avg_sq"] for s in sts],
                           [s["max_exp_avg_sq"] for s in sts] if self._amsgrad else None,
                           lp=self._lp(grp), lr=self.lr, beta1=b1, beta2=b2, eps=self._eps, wd=self._weight_decay,
                           bc1=bc1, bc2=bc2, adamw=self._DECOUPLED, amsgrad=self._amsgrad,
                           inv_scale=self._inv_scale, found_inf=self._found_inf, step_dev=step_dev)
        if step_dev is not None:
            self._advance_device_step()
        if rest and self._skip():
            self._step_count -= 1
            return
        for p in rest:
            st = self._state(p, names)
            g = self._grad(p)                              # may alias p.grad: never modified in place
            m, v = st["exp_avg"], st["exp_avg_sq"]
            with torch.no_grad():
                w = p if p.dtype == torch.float32 else p.float()      # fp32 parameters are updated in place
                if self._DECOUPLED:
                    if self._weight_decay:
                        w.mul_(1 - self.lr * self._weight_decay)
                elif self._weight_decay:
                    g = g + self._weight_decay * w
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                vv = v
                if self._amsgrad:
                    torch.maximum(st["max_exp_avg_sq"], v, out=st["max_exp_avg_sq"])
                    vv = st["max_exp_avg_sq"]
                denom = vv.sqrt().div_(bc2 ** 0.5).add_(self._eps)      # sqrt(v / bc2) + eps, one temporary
                w.addcdiv_(m, denom, value=-(self.lr / bc1))
                if w is not p:
                    p.copy_(w)
                lp = getattr(p, "_axon_lp", None)
                if lp is not None:
                    lp.copy_(p)


class AdamW(Adam):
    _DECOUPLED = True
    _DEFAULT_WD = 0.01
