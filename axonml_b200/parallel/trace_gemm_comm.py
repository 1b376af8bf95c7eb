"""Prints the per-tile timeline of the GEMM -> reduce-scatter kernel on rank 0 (multi-rank kernels
cannot run under a profiler, so the kernel stamps ``globaltimer`` itself when a trace buffer is set).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m axonml_b200.parallel.trace_gemm_comm [--tokens-per-rank 4096 --hidden 4096 --ffn 14336]
"""
from __future__ import annotations

import argparse
import ctypes
import os

import torch
import torch.distributed as dist


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens-per-rank", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    a = ap.parse_args(argv)
    from .. import _native as N
    from . import NcclBackend, ProcessGroup
    from .gemm_comm import FusedGemmComm
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    pg = ProcessGroup(NcclBackend.init(timeout_s=120))
    W, rank = pg.world_size(), pg.rank()
    eng = FusedGemmComm.try_create(pg)
    assert eng is not None, "symmetric memory is not available"
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    for K, name in ((a.hidden // W, "o_proj"), (a.ffn // W, "down")):
        x = torch.randn(a.tokens_per_rank * W, K, device="cuda").bfloat16()
        w = torch.randn(a.hidden, K, device="cuda").bfloat16() * 0.02
        for _ in range(3):
            eng.gemm_rs(x, w)
        torch.cuda.synchronize()
        dist.barrier()
        tr = torch.zeros(sms * 64, dtype=torch.int64, device="cuda")
        N.cuda().ax_gemm_comm_set_trace(ctypes.c_void_p(tr.data_ptr()))
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        eng.gemm_rs(x, w)
        e1.record()
        torch.cuda.synchronize()
        N.cuda().ax_gemm_comm_set_trace(ctypes.c_void_p(0))
        dist.barrier()
        if rank == 0:
            t = tr.cpu().view(sms, 64)
            t0 = int(t[:, 0][t[:, 0] > 0].min())
            print(f"== {name}: K = {K} per rank, {W} ranks: CUDA-event time {e0.elapsed_time(e1) * 1e3:.0f} us, "
                  f"kernel span {(int(t[:, 63].max()) - t0) / 1e3:.1f} us")

            def f(v):
                return f"{(int(v) - t0) / 1e3:7.1f}" if int(v) > 0 else "      -"
            for cta in (0, sms // 2, sms - 1):
                r = t[cta]
                print(f" CTA {cta}: start {f(r[0])}  start-of-call wait done {f(r[1])}  epilogues done {f(r[62])}  end {f(r[63])}")
                for it in range(15):
                    s = r[2 + 4 * it:6 + 4 * it]
                    if int(s[0]) == 0 and int(s[3]) == 0:
                        break
                    print(f"   tile {it:2d}: accumulator ready {f(s[0])}  peers' flags {f(s[1])}  epilogue done {f(s[2])}  "
                          f"MMA issued {f(s[3])}")
    dist.barrier()


if __name__ == "__main__":
    main()
