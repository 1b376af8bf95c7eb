"""The allocation-free norm backward (``ax_norm_bwd_noalloc``) against the regular entry point.

Callers that cannot allocate device memory at call time - inside a CUDA-graph capture, in a
serving loop where cudaMalloc would stall the GPU, or as a guest in another runtime's memory
arena - use the variant whose scratch is a fixed array inside the library.  This test calls it
through its exported C symbol (plain ctypes on the shared object, no wrapper) twice in a row, with
different shapes, and compares each result with ``ax_norm_bwd`` given a torch-allocated scratch.
The file name keeps it last in collection order.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "axonml_b200", "_lib",
                   "libaxonml_cuda.so")


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _reference(x, dy, w, rms, dres):
    """LayerNorm / RMSNorm backward written out in fp32 torch (autograd on the defining formula)."""
    xf = x.float().requires_grad_()
    wf = w.float().requires_grad_()
    bf = torch.zeros_like(wf).requires_grad_()
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    else:
        y = (xf - xf.mean(-1, keepdim=True)) * torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + 1e-5) * wf + bf
    y.backward(dy.float())
    dx = xf.grad + (dres.float() if dres is not None else 0)
    return dx, wf.grad, bf.grad


def _run_pair(lib, rows, D, rms, dtype, w_dtype=None, with_dres=False):
    dev = "cuda"
    w_dtype = w_dtype or dtype
    code = 1 if dtype == torch.bfloat16 else 0
    wcode = 1 if w_dtype == torch.bfloat16 else 0
    x = torch.randn(rows, D, device=dev).to(dtype)
    dy = torch.randn(rows, D, device=dev).to(dtype)
    w = (1 + 0.1 * torch.randn(D, device=dev)).to(w_dtype)
    dres = torch.randn(rows, D, device=dev).to(dtype) if with_dres else None
    xf = x.float()
    mean = torch.zeros(rows, device=dev) if rms else xf.mean(-1)
    var = xf.pow(2).mean(-1) if rms else xf.var(-1, unbiased=False)
    rstd = torch.rsqrt(var + 1e-5)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    groups = lib.ax_norm_bwd_groups(rows)
    scratch = torch.empty(groups * 2 * D, device=dev)
    dx0, dw0, db0 = torch.empty_like(x), torch.empty_like(w), torch.zeros_like(w)
    rc = lib.ax_norm_bwd(int(rms), code, wcode, _p(dy), _p(x), _p(w), _p(mean), _p(rstd), _p(dres),
                         _p(dx0), _p(dw0), _p(db0), _p(scratch), groups, rows, D, stream)
    assert rc == 0

    dx1, dw1, db1 = torch.empty_like(x), torch.empty_like(w), torch.zeros_like(w)
    rc = lib.ax_norm_bwd_noalloc(int(rms), code, wcode, _p(dy), _p(x), _p(w), _p(mean), _p(rstd),
                                 _p(dres), _p(dx1), _p(dw1), _p(db1), rows, D, stream)
    assert rc == 0
    torch.cuda.synchronize()
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    assert torch.allclose(dx1.float(), dx0.float(), **tol)
    wt = dict(atol=1e-3, rtol=2e-2) if w_dtype == torch.float32 else dict(atol=0.05 * rows ** 0.5, rtol=2e-2)
    assert torch.allclose(dw1.float(), dw0.float(), **wt)
    if not rms:
        assert torch.allclose(db1.float(), db0.float(), **wt)
    # and against the formula itself, not only against the sibling entry point
    rdx, rdw, rdb = _reference(x, dy, w, rms, dres)
    assert torch.allclose(dx1.float(), rdx, **(dict(atol=2e-3, rtol=2e-3) if dtype == torch.float32 else dict(atol=6e-2, rtol=4e-2)))
    wr = dict(atol=2e-3 * rows ** 0.5, rtol=2e-2) if w_dtype == torch.float32 else dict(atol=0.06 * rows ** 0.5, rtol=3e-2)
    assert torch.allclose(dw1.float(), rdw, **wr)
    if not rms:
        assert torch.allclose(db1.float(), rdb, **wr)


def test_noalloc_norm_backward_matches_regular_entry_twice():
    lib = ctypes.CDLL(LIB)
    # first call: many rows (uses all 64 slots); second: few rows, other D and dtype, so that any
    # stale partials left in the shared array by the first call would show up
    _run_pair(lib, 4096, 2048, False, torch.bfloat16)
    _run_pair(lib, 37, 512, True, torch.float32)


def test_noalloc_at_the_largest_width_with_residual_gradient_and_mixed_types():
    """The cases at the edge of the built-in scratch: D at the limit with enough rows to use every
    partial slot, a residual-stream gradient added to dx, and bf16 activations with fp32 weights.
    Two calls in a row again, the second smaller, so stale partials would show."""
    lib = ctypes.CDLL(LIB)
    max_d, max_g = ctypes.c_int(0), ctypes.c_int(0)
    assert lib.ax_norm_bwd_noalloc_limits(ctypes.byref(max_d), ctypes.byref(max_g)) == 0
    _run_pair(lib, 640, max_d.value, False, torch.bfloat16, with_dres=True)
    _run_pair(lib, 200, 1024, True, torch.bfloat16, w_dtype=torch.float32, with_dres=True)
    _run_pair(lib, 513, max_d.value, True, torch.float32)


def test_noalloc_rejects_oversize():
    lib = ctypes.CDLL(LIB)
    max_d, max_g = ctypes.c_int(0), ctypes.c_int(0)
    assert lib.ax_norm_bwd_noalloc_limits(ctypes.byref(max_d), ctypes.byref(max_g)) == 0
    D = max_d.value + 8
    t = torch.zeros(8, device="cuda")
    rc = lib.ax_norm_bwd_noalloc(0, 0, 0, _p(t), _p(t), _p(t), _p(t), _p(t), _p(None), _p(t), _p(t),
                                 _p(t), 1, D, ctypes.c_void_p(0))
    assert rc == -2
