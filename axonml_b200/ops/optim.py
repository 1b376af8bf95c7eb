"""Multi-tensor fused optimizer steps (``csrc/kernels/optim.cu``).

``multi_tensor(kind, params, grads, ...)`` packs raw pointers into ctypes arrays and issues one
native call; the native side splits the list into as few launches as the kernel-parameter table
allows.  All scalars that change every step (lr, bias corrections) are passed by value, the loss
scale and the found-inf flag by device pointer, so a step never synchronises with the host.  When
a device-side found-inf flag can skip a step, the step count used for Adam's and LAMB's bias
corrections is kept on the device too (``step_dev``) and only advances on steps that were taken.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as N

KIND = {"sgd": 0, "adam": 1, "rmsprop": 2, "lamb1": 3, "lamb2": 4, "sumsq": 5, "scale": 6,
        "unscale_check": 7}


def _ptr_array(tensors):
    if tensors is None:
        return None
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if t is not None else None
    return arr


def supported(params, grads) -> bool:
    if not N.have_gpu() or not params:
        return False
    pd, gd = params[0].dtype, grads[0].dtype
    ok = (torch.float32, torch.bfloat16)
    if pd not in ok or gd not in ok:
        return False
    for p, g in zip(params, grads):
        if not (p.is_cuda and g.is_cuda and p.dtype == pd and g.dtype == gd and p.is_contiguous()
                and g.is_contiguous()):
            return False
    return True


def multi_tensor(kind: str, params, grads, s1=None, s2=None, s3=None, lp=None, *, lr=0.0,
                 beta1=0.0, beta2=0.0, eps=0.0, wd=0.0, bc1=1.0, bc2=1.0, momentum=0.0,
                 dampening=0.0, alpha=0.0, nesterov=False, first_step=False, adamw=False,
                 amsgrad=False, centered=False, inv_scale=None, found_inf=None, norms=None,
                 clip_coef=None, step_dev=None) -> None:
    ref = params if params is not None else grads
    nt = len(ref)
    if nt == 0:
        return
    # the kernel refreshes bf16 mirrors itself; mirrors of another dtype are copied afterwards
    late_lp = None
    if lp is not None and any(l is not None and l.dtype != torch.bfloat16 for l in lp):
        late_lp, lp = lp, None
    p_bf16 = int(params is not None and params[0].dtype == torch.bfloat16)
    g_bf16 = int(grads is not None and grads[0].dtype == torch.bfloat16)
    sizes = (ctypes.c_long * nt)(*[t.numel() for t in ref])
    hyper = (ctypes.c_float * 10)(lr, beta1, beta2, eps, wd, bc1, bc2, momentum, dampening, alpha)
    flags = (ctypes.c_int * 5)(int(nesterov), int(first_step), int(adamw), int(amsgrad),
                               int(centered))
    rc = N.cuda().ax_multi_tensor(
        KIND[kind], p_bf16, g_bf16, nt, _ptr_array(params), _ptr_array(grads), _ptr_array(s1),
        _ptr_array(s2), _ptr_array(s3), _ptr_array(lp), sizes, hyper, flags, N.ptr(inv_scale),
        N.ptr(found_inf), N.ptr(norms), N.ptr(clip_coef), N.ptr(step_dev), N.stream_ptr())
    N.check(rc, f"ax_multi_tensor[{kind}]")
    if late_lp is not None and kind in ("sgd", "adam", "rmsprop", "lamb2"):
        for l, q in zip(late_lp, params):
            if l is not None:
                l.copy_(q)


def grad_sumsq(grads, out: torch.Tensor | None = None, inv_scale=None) -> torch.Tensor:
    """Sum of squares of all gradients into a 1-element fp32 tensor (no host sync)."""
    dev = grads[0].device
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=dev)
    if supported(grads, grads):
        multi_tensor("sumsq", None, grads, norms=out, inv_scale=inv_scale)
    else:
        s = sum((g.float() ** 2).sum() for g in grads)
        if inv_scale is not None:
            s = s * inv_scale.float() ** 2
        out += s
    return out
