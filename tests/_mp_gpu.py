"""Helper: run a function as N GPU ranks (NCCL, one process per GPU) in child processes."""
import os
import sys
import traceback

import torch
import torch.multiprocessing as mp

from tests._mp import _free_port, _plain, _unplain


def _entry(rank, world, port, fn, args, q, env):
    try:
        os.environ.update(env)
        os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world), str(rank)
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from axonml_b200.parallel import NcclBackend
        be = NcclBackend.init(rank, world, "127.0.0.1", port, timeout_s=60)
        out = fn(rank, world, be, *args)
        torch.cuda.synchronize()
        q.put((rank, "ok", _plain(out)))
        try:
            be.destroy()
        except Exception:
            pass
    except Exception as e:  # noqa: BLE001
        q.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


def run_gpu_ranks(fn, world: int = 2, args=(), env=None, timeout_s: float = 180.0):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q, dict(env or {})), daemon=True)
             for r in range(world)]
    [p.start() for p in procs]
    res = {}
    try:
        for _ in procs:
            r, st, val = q.get(timeout=timeout_s)
            res[r] = (st, _unplain(val))
    finally:
        # a rank that is stuck must not keep the test process alive
        for p in procs:
            p.join(10 if len(res) == len(procs) else 0.1)
            if p.is_alive():
                p.kill()
    for r, (st, val) in res.items():
        assert st == "ok", f"rank {r}: {val}"
    return res
