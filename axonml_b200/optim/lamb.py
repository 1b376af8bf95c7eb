"""LAMB (crates/axonml-optim/src/lamb.rs:105-280): Adam moments, update
``r = m_hat / (sqrt(v_hat) + eps) + wd*p``, layer-wise trust ratio ``|p| / |r|`` (1 when either
norm is 0), ``p -= lr * trust * r``.  Default eps 1e-6."""
from __future__ import annotations

import torch

from ..ops import optim as O
from .optimizer import Optimizer


class LAMB(Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-6,
                 weight_decay: float = 0.0, bias_correction: bool = True):
        super().__init__(params, lr)
        self._betas, self._eps, self._weight_decay = tuple(betas), eps, weight_decay
        self._bias_correction = bias_correction

    @classmethod
    def new(cls, params, lr): return cls(params, lr)

    @classmethod
    def with_betas(cls, params, lr, betas): return cls(params, lr, betas)

    @classmethod
    def with_options(cls, params, lr, betas, eps, weight_decay): return cls(params, lr, betas, eps, weight_decay)

    def betas(self, b1, b2): self._betas = (b1, b2); return self
    def eps(self, e): self._eps = e; return self
    def weight_decay(self, wd): self._weight_decay = wd; return self
    def bias_correction(self, flag=True): self._bias_correction = flag; return self

    def _hyper(self):
        return {"_betas": self._betas, "_eps": self._eps, "_weight_decay": self._weight_decay,
                "_bias_correction": self._bias_correction}

    @torch.no_grad()
    def step(self) -> None:
        self._step_count += 1
        t = self._step_count
        b1, b2 = self._betas
        bc1 = 1 - b1 ** t if self._bias_correction else 1.0
        bc2 = 1 - b2 ** t if self._bias_correction else 1.0
        names = ("exp_avg", "exp_avg_sq", "update")
        fused, rest = self._groups(self._active())
        for grp in fused:
            sts = [self._state(p, names) for p in grp]
            norms = torch.zeros(2 * len(grp), dtype=torch.float32, device=grp[0].device)
            hp = dict(lp=self._lp(grp), lr=self.lr, beta1=b1, beta2=b2, eps=self._eps, wd=self._weight_decay, bc1=bc1,
                      bc2=bc2, inv_scale=self._inv_scale, found_inf=self._found_inf, norms=norms)
            args = (grp, [self._g(p) for p in grp], [s["exp_avg"] for s in sts],
                    [s["exp_avg_sq"] for s in sts], [s["update"] for s in sts])
            O.multi_tensor("lamb1", *args, **hp)
            O.multi_tensor("lamb2", *args, **hp)
        if rest and self._skip():
            self._step_count -= 1
            return
        for p in rest:
            st = self._state(p, names[:2])
            g = self._grad(p)
            pf = p.float()
            m, v = st["exp_avg"], st["exp_avg_sq"]
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            r = (m / bc1) / ((v / bc2).sqrt() + self._eps) + self._weight_decay * pf
            pn, rn = pf.norm(), r.norm()
            trust = (pn / rn).item() if pn > 0 and rn > 0 else 1.0
            self._write(p, (pf - self.lr * trust * r).to(p.dtype))
