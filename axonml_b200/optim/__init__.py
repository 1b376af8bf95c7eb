"""Optimizers, GradScaler and LR schedulers (crates/axonml-optim)."""
from .adam import Adam, AdamW
from .grad_scaler import GradScaler, GradScalerState
from .lamb import LAMB
from .lr_scheduler import (CosineAnnealingLR, ExponentialLR, LRScheduler, MultiStepLR, OneCycleLR,
                           ReduceLROnPlateau, StepLR, WarmupLR)
from .optimizer import Optimizer, ParamState
from .rmsprop import RMSprop
from .sgd import SGD


def clip_grad_norm(params, max_norm: float, norm_type: float = 2.0):
    """Scales gradients so that their global L2 norm is at most ``max_norm``; returns the norm
    (crates/axonml/src/trainer.rs:413-440).  On CUDA the norm and the scaling are two
    multi-tensor launches with no host synchronisation."""
    import torch
    from ..ops import optim as O
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return torch.zeros(())
    if norm_type == 2.0 and grads[0].is_cuda and all(g.dtype == grads[0].dtype for g in grads) and O.supported(grads, grads):
        ss = O.grad_sumsq(grads)
        norm = ss.sqrt()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        O.multi_tensor("scale", None, grads, clip_coef=coef)
        return norm[0]
    norm = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g.float(), norm_type) for g in grads]), norm_type)
    coef = float(max_norm) / (float(norm) + 1e-6)
    if coef < 1.0:
        for g in grads:
            g.mul_(coef)
    return norm


def clip_grad_value(params, clip_value: float) -> None:
    for p in params:
        if p.grad is not None:
            p.grad.clamp_(-clip_value, clip_value)
