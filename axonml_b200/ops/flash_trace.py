"""Prints the softmax-stage timeline of the flash-attention forward kernel: the kernel stamps
``globaltimer`` per KV block in one warp of two CTAs when a trace buffer is set.

    python -m axonml_b200.ops.flash_trace [--batch 4 --seq 2048 --heads 16]
"""
from __future__ import annotations

import argparse
import ctypes

import torch


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    a = ap.parse_args(argv)
    from .. import _native as N
    from .flash import flash_attention
    q, k, v = (torch.randn(a.batch, a.seq, a.heads, 128, device="cuda").bfloat16() for _ in range(3))
    with torch.no_grad():
        for _ in range(3):
            flash_attention(q, k, v, True)
        torch.cuda.synchronize()
        tr = torch.zeros(2 * 128, dtype=torch.int64, device="cuda")
        N.cuda().ax_flash_fwd_set_trace(ctypes.c_void_p(tr.data_ptr()))
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        flash_attention(q, k, v, True)
        e1.record()
        torch.cuda.synchronize()
        N.cuda().ax_flash_fwd_set_trace(ctypes.c_void_p(0))
    print(f"CUDA-event time of the traced launch: {e0.elapsed_time(e1) * 1e3:.1f} us")
    t = tr.cpu().view(2, 128)
    for c in range(2):
        r = t[c]
        t0 = int(r[0])
        if t0 == 0:
            continue
        print(f"CTA {c}: epilogue done at {(int(r[127]) - t0) / 1e3:.2f} us")
        prev = t0
        for j in range(25):
            s = [int(x) for x in r[1 + 5 * j:6 + 5 * j]]
            if len(s) < 5 or s[0] == 0:
                break
            print(f"  block {j:2d}: S ready +{(s[0] - prev) / 1e3:5.2f} | in registers +{(s[1] - s[0]) / 1e3:5.2f} | "
                  f"max/rescale +{(s[2] - s[1]) / 1e3:5.2f} | P buffer +{(s[3] - s[2]) / 1e3:5.2f} | "
                  f"exp+store +{(s[4] - s[3]) / 1e3:5.2f}   (t = {(s[4] - t0) / 1e3:6.2f} us)")
            prev = s[4]


if __name__ == "__main__":
    main()
