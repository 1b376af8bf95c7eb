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

    # A parameter may be one rank's slice of a flat buffer that holds several tensors (the master
    # shard of a sharded engine).  The engine then attaches ``_axon_segments`` = [(tensor id,
    # start, length)] and ``_axon_norm_reduce`` (sums a tensor over the ranks that hold the other
    # slices): the trust ratio is taken per tensor over all its slices, not per slice.
    def _pieces(self, ps, names):
        out = []
        for p in ps:
            st = self._state(p, names)
            g, lp = self._g(p), getattr(p, "_axon_lp", None)
            segs = getattr(p, "_axon_segments", None)
            if segs is None:
                out.append((p, g, st["exp_avg"], st["exp_avg_sq"], st["update"], lp, None))
                continue
            pf, gf = p.detach().view(-1), g.view(-1)
            for gid, s, n in segs:
                if n > 0:
                    e = s + n
                    out.append((pf[s:e], gf[s:e], st["exp_avg"].view(-1)[s:e], st["exp_avg_sq"].view(-1)[s:e],
                                st["update"].view(-1)[s:e], None if lp is None else lp.view(-1)[s:e], gid))
        return out

    @staticmethod
    def _reduce_norms(norms, pieces, reducers):
        """``norms`` [pieces, 2] local sums of squares -> sums over every slice of the same tensor."""
        gids = [pc[6] for pc in pieces]
        if not reducers or all(i is None for i in gids):
            return norms
        total = max(r[1] for r in reducers)
        rows = [k for k, i in enumerate(gids) if i is not None]
        idx = torch.tensor([gids[k] for k in rows], dtype=torch.long, device=norms.device)
        sel = torch.tensor(rows, dtype=torch.long, device=norms.device)
        glob = torch.zeros(total, 2, dtype=torch.float32, device=norms.device)
        glob.index_add_(0, idx, norms[sel])
        reducers[0][0](glob)
        norms = norms.clone()
        norms[sel] = glob[idx]
        return norms

    @torch.no_grad()
    def step(self) -> None:
        self._step_count += 1
        t = self._step_count
        b1, b2 = self._betas
        bc1 = 1 - b1 ** t if self._bias_correction else 1.0
        bc2 = 1 - b2 ** t if self._bias_correction else 1.0
        names = ("exp_avg", "exp_avg_sq", "update")
        active = self._active()
        reducers = [(p._axon_norm_reduce, p._axon_num_tensors) for p in active
                    if getattr(p, "_axon_norm_reduce", None) is not None]
        fused, rest = self._groups(active)
        if reducers and len(fused) + bool(rest) > 1:          # one reduction per step: keep the slices together
            fused, rest = ([[p for grp in fused for p in grp]], rest) if not rest else ([], active)
        step_dev = self._device_step(fused[0][0].device) if (fused and self._bias_correction) else None
        for grp in fused:
            pcs = self._pieces(grp, names)
            norms = torch.zeros(len(pcs), 2, dtype=torch.float32, device=grp[0].device)
            lps = [pc[5] for pc in pcs]
            hp = dict(lp=lps if any(l is not None for l in lps) else None, lr=self.lr, beta1=b1, beta2=b2,
                      eps=self._eps, wd=self._weight_decay, bc1=bc1, bc2=bc2, inv_scale=self._inv_scale,
                      found_inf=self._found_inf, norms=norms, step_dev=step_dev)
            args = ([pc[0] for pc in pcs], [pc[1] for pc in pcs], [pc[2] for pc in pcs], [pc[3] for pc in pcs],
                    [pc[4] for pc in pcs])
            O.multi_tensor("lamb1", *args, **hp)
            hp["norms"] = self._reduce_norms(norms, pcs, reducers)
            O.multi_tensor("lamb2", *args, **hp)
        if step_dev is not None:
            self._advance_device_step()
        if rest and self._skip():
            self._step_count -= 1
            return
        if rest:
            pcs = self._pieces(rest, names)
            norms = torch.zeros(len(pcs), 2, dtype=torch.float32, device=rest[0].device)
            for k, (pv, gv, m, v, r, _, _) in enumerate(pcs):
                g = gv.float()
                if self._inv_scale is not None:
                    g = g * self._inv_scale.to(g.device)
                pf = pv.float()
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                r.copy_((m / bc1) / ((v / bc2).sqrt() + self._eps) + self._weight_decay * pf)
                norms[k, 0] = (pf * pf).sum()
                norms[k, 1] = (r * r).sum()
            norms = self._reduce_norms(norms, pcs, reducers).sqrt()
            for k, (pv, _, _, _, r, lp, _) in enumerate(pcs):
                pn, rn = norms[k, 0], norms[k, 1]
                trust = torch.where((pn > 0) & (rn > 0), pn / rn.clamp_min(1e-30), torch.ones_like(pn))
                pv.sub_((self.lr * trust * r).to(pv.dtype))
                if lp is not None:
                    lp.copy_(pv)
