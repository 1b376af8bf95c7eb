"""fp32 master weights for models whose parameters live in bf16.

``MasterParams(model.parameters())`` keeps one fp32 copy per low-precision parameter.  The copies
are what the optimizer owns (moments are fp32 too); after every step the fused multi-tensor
kernels write the updated value to the master AND to the bf16 parameter in the same pass
(``_axon_lp``), and they read the bf16 gradient directly (``_axon_grad``), so no cast kernels run.

This is the replicated-parameter counterpart of what the sharded engine (``parallel/fsdp.py``) does
for its shards; the reference documents the intent in its AMP notes (crates/axonml/src/lib.rs:37-47,
crates/axonml-autograd/src/amp.rs:80-140) but never wires master weights up.
"""
from __future__ import annotations

import torch


class MasterParams:
    def __init__(self, params):
        self.low = [p for p in params]
        self.master = []
        for p in self.low:
            m = p.detach().float().clone() if p.dtype != torch.float32 else p.detach()
            if p.dtype != torch.float32:
                m._axon_lp = p.data
            self.master.append(m)

    def parameters(self):
        return self.master

    def attach_grads(self) -> None:
        """Call after backward: hands the low-precision gradients to the optimizer."""
        for m, p in zip(self.master, self.low):
            m._axon_grad = p.grad

    def zero_grad(self) -> None:
        for m, p in zip(self.master, self.low):
            p.grad = None
            m._axon_grad = None

    def state_dict(self) -> dict:
        return {"master": [m.detach().clone() for m in self.master]}

    def load_state_dict(self, sd: dict) -> None:
        with torch.no_grad():
            for m, src, p in zip(self.master, sd["master"], self.low):
                m.copy_(src)
                if m is not p:
                    p.copy_(m)
