"""Bandwidth of the peer-memory paths the fused collectives are built on: bulk and per-thread
stores to the next rank's symmetric buffer for several grid sizes, and loads of peer-written
symmetric memory in four flavours (``ld.relaxed.sys``, ``ld.global.cg``, plain, ``ld.relaxed.gpu``).
CUDA-event timings, every rank stores to rank+1 at the same time.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m axonml_b200.parallel.bench_peer_copy
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist


def main() -> None:
    from .. import _native as N
    from . import NcclBackend, ProcessGroup
    from .symm import SymmetricHeap
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    pg = ProcessGroup(NcclBackend.init(timeout_s=120))
    heap = SymmetricHeap(pg)
    rank, W = heap.rank, heap.world
    L, st = N.cuda(), N.stream_ptr()
    total = 256 << 20
    buf = heap.allocate(total, torch.uint8)
    peer, local = buf.peer_ptrs[(rank + 1) % W], buf.peer_ptrs[rank]

    def store(target, grid, threads, piece, depth, mode):
        unit = max(piece, 16) * (threads // 32) * 16
        per = (total // grid) // unit * unit
        for _ in range(2):
            N.check(L.ax_peer_store_bench(ctypes.c_void_p(target), ctypes.c_long(per), piece, depth, mode, grid, threads, st), "store")
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        for _ in range(5):
            L.ax_peer_store_bench(ctypes.c_void_p(target), ctypes.c_long(per), piece, depth, mode, grid, threads, st)
        e1.record()
        torch.cuda.synchronize()
        return per * grid * 5 / (e0.elapsed_time(e1) * 1e-3) / 1e9

    rows = []
    for grid in (16, 32, 74, 148):
        for piece, depth, threads in ((4096, 8, 128), (16384, 8, 128), (16384, 8, 32)):
            rows.append((f"bulk store  grid {grid:3d}  piece {piece:5d}  {threads // 32} warp(s)", store(peer, grid, threads, piece, depth, 0)))
        rows.append((f"st.v4       grid {grid:3d}  128 threads", store(peer, grid, 128, 4096, 1, 1)))
    rows.append(("bulk store to LOCAL memory, grid 148, piece 4096", store(local, 148, 128, 4096, 8, 0)))
    # loads: the peer fills this rank's buffer first, so the lines were last written over NVLink
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    span = sms << 20
    view = buf.peer_tensor((rank + 1) % W, (span,), torch.uint8)
    sink = torch.zeros(4, dtype=torch.int32, device="cuda")
    ns = torch.zeros(sms, dtype=torch.int64, device="cuda")
    names = ["ld.relaxed.sys", "ld.global.cg", "ld.global", "ld.relaxed.gpu"]
    L.ax_peer_load_bench(2, ctypes.c_void_p(local), ctypes.c_long(1 << 20), N.ptr(sink), N.ptr(ns), sms, st)   # warm-up
    for flavour, name in enumerate(names):
        view.fill_(flavour + 1)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        N.check(L.ax_peer_load_bench(flavour, ctypes.c_void_p(local), ctypes.c_long(1 << 20), N.ptr(sink), N.ptr(ns), sms, st), "load")
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3
        rows.append((f"{name:15s} of peer-written symmetric memory: {float(ns.float().mean()) / 64 / 1e3:5.2f} us per 4 KB piece per warp",
                     span / us / 1e3))
        dist.barrier()
    if rank == 0:
        for name, v in rows:
            print(f"{name:90s} {v:8.1f} GB/s", flush=True)
    dist.barrier()


if __name__ == "__main__":
    main()
