"""Times the fused tensor-parallel kernels against their composed baseline and their roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P -m axonml_b200.parallel.bench_gemm_comm [--tokens-per-rank 4096] [--iters 20]

For every projection of the Llama-8B block at tensor-parallel size N it reports, per launch (CUDA
events on the launching stream, max over ranks, inputs far larger than L2 rotated between
iterations): the fused kernel, the composed path (NCCL collective + plain tcgen05 GEMM) and the
roofline = the slower of FLOPs / measured GEMM peak and NVLink bytes / measured link bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _peaks():
    tflops, link = 1590.0, 770.0          # fallback: earlier measurement on the same pool
    src = "fallback"
    for base in (os.getcwd(), os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))):
        p = os.path.join(base, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            try:
                d = json.load(open(p))
                tflops = float(d.get("bf16_tflops", tflops))
                src = "measured"
            except Exception:
                pass
            break
    return tflops, link, src


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens-per-rank", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--only", default="", help="comma-separated substrings of the rows to run")
    args = ap.parse_args()
    from axonml_b200 import _native
    from axonml_b200.ops.gemm import gemm_bf16
    from axonml_b200.parallel import NcclBackend, ProcessGroup
    from axonml_b200.parallel.gemm_comm import FusedGemmComm
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    pg = ProcessGroup(NcclBackend.init(timeout_s=300))
    W, rank = pg.world_size(), pg.rank()
    eng = FusedGemmComm.try_create(pg)
    assert eng is not None, "symmetric memory is not available"
    tflops, link, src = _peaks()
    H, hd, tl = args.hidden, args.hidden // args.heads, args.tokens_per_rank
    T = tl * W
    qkv_n, ffn2 = (args.heads + 2 * args.kv_heads) * hd // W, 2 * args.ffn // W
    # (name, kind, K, N, weight given as [N, K]); the last four are the input-gradient launches of the
    # same layers: the weight is then read as [K, N] and the roles of the two kernels swap
    shapes = [("qkv  all-gather->GEMM", "ag", H, qkv_n, True),
              ("gate|up all-gather->GEMM", "ag", H, ffn2, True),
              ("o_proj GEMM->reduce-scatter", "rs", args.heads * hd // W, H, True),
              ("down   GEMM->reduce-scatter", "rs", args.ffn // W, H, True),
              ("qkv dgrad GEMM->reduce-scatter", "rs", qkv_n, H, False),
              ("gate|up dgrad GEMM->reduce-sc.", "rs", ffn2, H, False),
              ("o_proj dgrad all-gather->GEMM", "ag", H, args.heads * hd // W, False),
              ("down dgrad all-gather->GEMM", "ag", H, args.ffn // W, False)]
    if args.only:
        shapes = [sh for sh in shapes if any(o in sh[0] for o in args.only.split(","))]
    rows = []
    NB = 4                                            # rotating operand sets (weights + activations > L2)
    for name, kind, K, Nn, tb in shapes:
        ws = [(torch.randn((Nn, K) if tb else (K, Nn), device="cuda") * 0.02).bfloat16() for _ in range(NB)]
        if kind == "ag":
            xs = [torch.randn(tl, K, device="cuda").bfloat16() for _ in range(NB)]
            gathered = torch.empty(W, tl, K, device="cuda", dtype=torch.bfloat16)
            ch = None if tb else eng.ag_bwd
            fused = lambda i: eng.ag_gemm(xs[i % NB], ws[i % NB], trans_b=tb, channel=ch)
            def composed(i):
                dist.all_gather_into_tensor(gathered, xs[i % NB])
                return gemm_bf16(gathered.view(T, K), ws[i % NB], trans_b=tb)
        else:
            xs = [torch.randn(T, K, device="cuda").bfloat16() for _ in range(NB)]
            outb = torch.empty(tl, Nn, device="cuda", dtype=torch.bfloat16)
            fused = lambda i: eng.gemm_rs(xs[i % NB], ws[i % NB], trans_b=tb)
            def composed(i):
                dist.reduce_scatter_tensor(outb, gemm_bf16(xs[i % NB], ws[i % NB], trans_b=tb))
                return outb

        def timeit(fn):
            for i in range(3):
                fn(i)
            torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.iters):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) * 1e3        # us

        t_f, t_c = timeit(fused), timeit(composed)
        _native.check_status()
        flops = 2.0 * T * K * Nn
        wire = (W - 1) / W * T * (K if kind == "ag" else Nn) * 2        # bytes in (AG) / out (RS) per GPU
        roof = max(flops / (tflops * 1e12), wire / (link * 1e9)) * 1e6
        rows.append((name, T, K, Nn, t_f, t_c, roof, roof / t_f))
    if rank == 0:
        print(f"tensor-parallel size {W}, {tl} tokens per rank; roofline denominators: {tflops:.0f} TFLOP/s bf16 ({src}), "
              f"{link:.0f} GB/s per direction NVLink (measured peer copy)")
        print(f"{'op':31s} {'M':>6s} {'K':>6s} {'N':>6s} {'fused us':>9s} {'nccl+gemm us':>12s} {'roofline us':>11s} {'frac':>5s}")
        for r in rows:
            print(f"{r[0]:31s} {r[1]:6d} {r[2]:6d} {r[3]:6d} {r[4]:9.1f} {r[5]:12.1f} {r[6]:11.1f} {r[7]:5.2f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
