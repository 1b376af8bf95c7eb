"""Stand-alone timing of the hand-written kernels on one GPU, with the achieved fraction of the
measured roofline (copy bandwidth / cuBLAS bf16 throughput from ``MEASURED_PEAKS.json`` when that
file is present in the working directory, else the stated fallback figures).

    python -m axonml_b200.benchmark_kernels gemm flash_fwd rmsnorm      # chosen workloads
    python -m axonml_b200.benchmark_kernels all --iters 20
    python -m axonml_b200.benchmark_kernels gemm_shapes                 # tile policies against cuBLAS
    python -m axonml_b200.benchmark_kernels gemv_shapes                 # decode matrix-vector kernels, both layouts
    python -m axonml_b200.benchmark_kernels flash_timeline              # in-kernel timeline of the flash forward
    python -m axonml_b200.benchmark_kernels gemm --small                # a few launches on a small case
                                                                        # (what a profiler capture uses)

Timing: CUDA events on the launching stream, 3 warm-up launches, operands rotated through more
memory than the 126 MB L2 between launches.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    hbm, tflops, src = 6650.0, 1590.0, "fallback"
    p = os.path.join(os.getcwd(), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            hbm, tflops, src = float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
        except Exception:
            pass
    return hbm, tflops, src


def _time(fn, iters):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3          # us


def _time_graph(fn, iters):
    """Device time per call of a short launch sequence: ``iters`` calls are captured in one CUDA graph
    and the graph is timed, so that the host's launch rate does not bound the result."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3          # us


def w_gemm(small):
    from .ops.gemm import gemm_bf16
    n = 2048 if small else 8192
    nb = 2 if small else 3
    a = [torch.randn(n, n, device="cuda").bfloat16() for _ in range(nb)]
    b = [torch.randn(n, n, device="cuda").bfloat16() for _ in range(nb)]
    return (lambda i: gemm_bf16(a[i % nb], b[i % nb])), 2.0 * n ** 3, 3 * n * n * 2, f"bf16 GEMM {n}^3"


def w_flash_fwd(small, bwd=False):
    from .ops import flash
    B, H, S, D = (2, 8, 1024, 128) if small else (4, 16, 2048, 128)
    nb = 2 if small else 4
    qs = [[torch.randn(B, S, H, D, device="cuda").bfloat16().requires_grad_(bwd) for _ in range(3)] for _ in range(nb)]
    flops = 4.0 * B * H * S * S * D / 2 * (3.5 if bwd else 1.0)
    if not bwd:
        return (lambda i: flash.flash_attention(*qs[i % nb], causal=True)), flops, 4 * B * S * H * D * 2, f"flash fwd B{B} H{H} S{S} D{D} causal"
    g = torch.randn(B, S, H, D, device="cuda").bfloat16()

    def run(i):
        q, k, v = qs[i % nb]
        q.grad = k.grad = v.grad = None
        flash.flash_attention(q, k, v, causal=True).backward(g)
    return run, flops, 8 * B * S * H * D * 2, f"flash fwd+bwd B{B} H{H} S{S} D{D} causal"


def w_flash_bwd_only(small):
    """The three backward launches alone (delta pre-pass, dK/dV, dQ), without autograd."""
    import math
    from .ops import flash
    B, H, S, D = (2, 8, 1024, 128) if small else (4, 16, 2048, 128)
    nb = 2 if small else 4
    sets = []
    for _ in range(nb):
        q, k, v = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(3))
        out, lse, _ = flash.flash_fwd(q, k, v, True, 1.0 / math.sqrt(D))
        sets.append((q, k, v, out, lse, torch.randn_like(out), torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)))

    def run(i):
        q, k, v, out, lse, g, dq, dk, dv = sets[i % nb]
        flash.flash_bwd(q, k, v, out, g, lse, True, 1.0 / math.sqrt(D), dq, dk, dv)
    flops = 4.0 * B * H * S * S * D / 2 * 2.5
    return run, flops, 8 * B * S * H * D * 2, f"flash bwd only B{B} H{H} S{S} D{D} causal"


def w_rmsnorm(small):
    from .ops import norm
    rows, D = (8192, 4096) if small else (65536, 4096)
    nb = 2 if small else 3
    xs = [torch.randn(rows, D, device="cuda").bfloat16() for _ in range(nb)]
    w = torch.ones(D, device="cuda").bfloat16()
    return (lambda i: norm.rms_norm(xs[i % nb], w, 1e-5)), 0.0, 2 * rows * D * 2, f"RMSNorm fwd [{rows}, {D}] bf16"


def w_adamw(small):
    from .ops import optim as O
    n = (8 if small else 64) * 1024 * 1024
    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda").bfloat16()
    m, v, lp = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda").bfloat16()

    def run(i):
        O.multi_tensor("adam", [p], [g], [m], [v], None, lp=[lp], lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1,
                       bc1=0.1, bc2=0.05, adamw=True, amsgrad=False, inv_scale=None, found_inf=None)
    return run, 0.0, n * (4 + 2 + 4 + 4) + n * (4 + 4 + 4 + 2), f"fused AdamW step, {n >> 20} Mi parameters (fp32 master, bf16 grad + mirror)"


def w_conv(small):
    from .ops import conv_igemm as CI
    n, c, h = (32, 128, 28) if small else (256, 128, 28)
    x = torch.randn(n, c, h, h, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w = CI._ohwi(torch.randn(c, c, 3, 3, device="cuda") * 0.05)
    return (lambda i: CI.fprop(x, w, None, (1, 1))), 2.0 * n * h * h * c * c * 9, 2 * n * h * h * c * 2, f"conv3x3 s1 fprop N{n} C{c} {h}x{h} NHWC bf16"


def w_qgemm(small):
    from .ops.quant import qgemm, tile_weight
    from .quant.quantize import quantize_tensor
    from .quant.types import QuantType
    Nn, K = (4096, 4096) if small else (28672, 4096)
    nb = 2 if small else 4
    ws = [tile_weight(quantize_tensor(torch.randn(Nn, K, device="cuda") * 0.02, QuantType.Q4_K)) for _ in range(nb)]
    x = torch.randn(1, K, device="cuda").bfloat16()
    return (lambda i: qgemm(x, ws[i % nb])), 0.0, Nn * K * 0.5625, f"Q4_K dequantising matmul batch 1, [{Nn}, {K}]"


def gemv_shapes(iters):
    """The four Q4_K projections of a Llama-3-8B layer at batch 1 in both weight layouts, and the
    Q8_0 head: device time and fraction of the measured copy bandwidth."""
    from .ops.quant import qgemm, tile_weight
    from .quant.quantize import quantize_tensor
    from .quant.types import QuantType
    gbs, _, src = _peaks()
    for name, Nn, K in (("qkv", 6144, 4096), ("o", 4096, 4096), ("gate|up", 28672, 4096), ("down", 4096, 14336),
                        ("qkv tp8", 768, 4096), ("o tp8", 4096, 512), ("gate|up tp8", 3584, 4096), ("down tp8", 4096, 1792)):
        nb = max(2, min(8, (400 << 20) // int(Nn * K * 0.5625) + 1))
        ws = [quantize_tensor(torch.randn(Nn, K, device="cuda") * 0.02, QuantType.Q4_K) for _ in range(nb)]
        x = torch.randn(1, K, device="cuda").bfloat16()
        line = f"{name:12s} [{Nn:6d}, {K:6d}]"
        for layout, mats in (("row-major", ws), ("tile128", [tile_weight(w) for w in ws])):
            us = _time_graph(lambda i: qgemm(x, mats[i % nb], out_dtype=torch.bfloat16), iters)
            tb = Nn * K * 0.5625 / us / 1e6
            line += f"  {layout}: {us:6.1f} us {tb:5.2f} TB/s ({tb * 1000 / gbs:.2f} of {src})"
        print(line, flush=True)


def flash_timeline(blocks: int = 8):
    """In-kernel timeline of the two-tile flash forward (the kernel stamps ``globaltimer`` when a
    trace buffer is set): per KV block of the first, longest CTA the softmax warps of tile A and
    tile B record when the scores are ready, in registers, the row maximum is known, the
    exponentials are done and the probabilities are stored."""
    import ctypes
    from .ops.flash import flash_attention
    q, k, v = (torch.randn(4, 2048, 16, 128, device="cuda").bfloat16() for _ in range(3))
    with torch.no_grad():
        for _ in range(3):
            flash_attention(q, k, v, True)
        torch.cuda.synchronize()
        tr = torch.zeros(4 * 128, dtype=torch.int64, device="cuda")
        _native.cuda().ax_flash_fwd_set_trace(ctypes.c_void_p(tr.data_ptr()))
        try:
            flash_attention(q, k, v, True)
            torch.cuda.synchronize()
        finally:
            _native.cuda().ax_flash_fwd_set_trace(ctypes.c_void_p(0))
    t = tr.cpu().view(4, 128)
    for tile in range(2):
        r = [int(x) for x in t[tile]]
        if r[0] == 0:
            continue
        print(f"tile {'AB'[tile]}: softmax loop done {(r[127] - r[0]) / 1e3:.2f} us after the CTA's start")
        prev = r[0]
        for j in range(blocks):
            s = r[1 + 5 * j:6 + 5 * j]
            if s[0] == 0:
                break
            print(f"  block {j:2d}: wait for scores {(s[0] - prev) / 1e3:5.2f} | TMEM load {(s[1] - s[0]) / 1e3:5.2f} | "
                  f"max / rescale {(s[2] - s[1]) / 1e3:5.2f} | exponentials {(s[3] - s[2]) / 1e3:5.2f} | "
                  f"store + arrive {(s[4] - s[3]) / 1e3:5.2f}  (us)")
            prev = s[4]


def w_paged(small):
    from .ops import paged
    B, ctx, Hq, Hkv, D, page = (8, 512, 32, 8, 128, 16) if small else (64, 768, 32, 8, 128, 16)
    pages = B * (ctx // page)
    kc = torch.randn(pages, page, Hkv, D, device="cuda").bfloat16()
    vc = torch.randn(pages, page, Hkv, D, device="cuda").bfloat16()
    table = torch.arange(pages, device="cuda", dtype=torch.int32).view(B, -1)
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    return (lambda i: paged.decode_attention(q, kc, vc, table, lens, page)), 0.0, 2 * B * ctx * Hkv * D * 2, f"paged decode attention B{B} ctx{ctx} GQA {Hq}/{Hkv}"


def w_flash_fwd_one_tile(small):
    from .ops import flash
    fn, flops, nbytes, desc = w_flash_fwd(small)

    def run(i):
        flash.set_one_tile(True)
        try:
            return fn(i)
        finally:
            flash.set_one_tile(False)
    return run, flops, nbytes, desc + " (one query tile per CTA)"


WORKLOADS = {"gemm": w_gemm, "flash_fwd": w_flash_fwd, "flash_fwd_one_tile": w_flash_fwd_one_tile, "flash_bwd": lambda s: w_flash_fwd(s, True), "flash_bwd_only": w_flash_bwd_only, "rmsnorm": w_rmsnorm,
             "adamw": w_adamw, "conv": w_conv, "qgemm": w_qgemm, "paged_decode": w_paged}


GEMM_SHAPES = [
    # (name, M, N, K, trans_a, trans_b): the Linear layers of the GPT-1.3B step (8192 tokens) in
    # forward, data-gradient and weight-gradient form, and the square case.
    ("square 8192", 8192, 8192, 8192, False, True),
    ("qkv fwd", 8192, 6144, 2048, False, True),
    ("proj fwd", 8192, 2048, 2048, False, True),
    ("fc1 fwd", 8192, 8192, 2048, False, True),
    ("fc2 fwd", 8192, 2048, 8192, False, True),
    ("head fwd", 8192, 50304, 2048, False, True),
    ("qkv dgrad", 8192, 2048, 6144, False, False),
    ("fc1 dgrad", 8192, 2048, 8192, False, False),
    ("fc2 dgrad", 8192, 8192, 2048, False, False),
    ("head dgrad", 8192, 2048, 50304, False, False),
    ("qkv wgrad", 6144, 2048, 8192, True, False),
    ("proj wgrad", 2048, 2048, 8192, True, False),
    ("fc1 wgrad", 8192, 2048, 8192, True, False),
    ("fc2 wgrad", 2048, 8192, 8192, True, False),
    ("head wgrad", 50304, 2048, 8192, True, False),
]


def gemm_shapes(iters):
    """Every tile policy of the GEMM kernel against ``torch.matmul`` (cuBLAS) on the Linear shapes of
    the GPT-1.3B step.  Operands rotate through more than the L2 capacity between launches."""
    from .ops.gemm import gemm_bf16, set_pair_mode
    from .ops.gemm import pair_capacity
    _, tflops, src = _peaks()
    print(f"CTA pairs resident at once: {pair_capacity()}")
    print(f"shape: cuBLAS us | one CTA bn128, bn256 | CTA pair bn128, bn256 | chosen -> TFLOP/s, of {src} peak, of cuBLAS")
    for name, M, N, K, ta, tb in GEMM_SHAPES:
        per = (M * K + N * K + M * N) * 2
        nb = max(2, min(6, (300 << 20) // per + 1))
        A = [torch.randn((K, M) if ta else (M, K), device="cuda").bfloat16() for _ in range(nb)]
        B = [torch.randn((N, K) if tb else (K, N), device="cuda").bfloat16() for _ in range(nb)]
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

        def ref(i):
            a = A[i % nb].t() if ta else A[i % nb]
            b = B[i % nb].t() if tb else B[i % nb]
            torch.matmul(a, b, out=out)
        t_ref = _time(ref, iters)
        ts = []
        for mode, bn in ((0, 128), (0, 256), (1, 128), (1, 256), (-1, 0)):
            set_pair_mode(mode)
            ts.append(_time(lambda i: gemm_bf16(A[i % nb], B[i % nb], trans_a=ta, trans_b=tb, out=out, bn=bn), iters))
        set_pair_mode(-1)
        fl = 2.0 * M * N * K
        print(f"{name} [{M}x{N}x{K}]: {t_ref:.1f} | {ts[0]:.1f}, {ts[1]:.1f} | {ts[2]:.1f}, {ts[3]:.1f} | {ts[4]:.1f} -> "
              f"{fl / ts[4] / 1e6:.0f} TFLOP/s, {fl / ts[4] / 1e6 / tflops:.2f}, {t_ref / ts[4]:.2f}", flush=True)
        del A, B, out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("names", nargs="+")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true", help="small case, three launches (for a profiler capture)")
    a = ap.parse_args()
    from . import _native
    if a.names == ["gemm_shapes"]:
        gemm_shapes(a.iters)
        _native.check_status()
        return
    if a.names == ["flash_timeline"]:
        flash_timeline()
        _native.check_status()
        return
    if a.names == ["gemv_shapes"]:
        gemv_shapes(a.iters)
        _native.check_status()
        return
    names = list(WORKLOADS) if a.names == ["all"] else a.names
    hbm, tflops, src = _peaks()
    print(f"roofline denominators ({src}): {hbm:.0f} GB/s copy, {tflops:.0f} TFLOP/s bf16")
    for n in names:
        fn, flops, nbytes, desc = WORKLOADS[n](a.small)
        if a.small:
            for i in range(3):
                fn(i)
            torch.cuda.synchronize()
            print(f"{n}: {desc}: 3 launches done")
            continue
        us = _time(fn, a.iters)
        _native.check_status()
        roof = max(flops / (tflops * 1e12), nbytes / (hbm * 1e9)) * 1e6
        kind = "compute" if flops / (tflops * 1e12) > nbytes / (hbm * 1e9) else "memory"
        rate = f"{flops / us / 1e6:.0f} TFLOP/s" if kind == "compute" else f"{nbytes / us / 1e3:.0f} GB/s"
        print(f"{n}: {desc}: {us:.1f} us, {rate}, {roof / us:.2f} of {src} {kind} roofline")


if __name__ == "__main__":
    main()
