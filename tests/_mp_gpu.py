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
    """Runs ``fn(rank, world, backend, *args)`` in one child process per GPU and returns
    ``{rank: (status, value)}``.

    A rank is never ended from outside while its buffers may be bound to an NVLink multicast
    object (``AXONML_NVLS`` not "0"): the ranks leave on their own.  That always happens in
    bounded time, because every device-side wait has a time budget (1 to 2 s) and the process
    group ends a collective whose partner is missing after 60 s.  Only when NVLS is off is a
    rank that is still alive after all of that killed, as a last resort."""
    env = dict(env or {})
    nvls_off = env.get("AXONML_NVLS", os.environ.get("AXONML_NVLS", "1")) == "0"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q, env), daemon=False)
             for r in range(world)]
    [p.start() for p in procs]
    res = {}
    # one failed rank makes the others run into the 60 s process-group timeout: leave room for it
    grace = 60.0 + 30.0
    try:
        import queue as _queue
        import time as _time
        deadline = _time.monotonic() + timeout_s
        while len(res) < world:
            left = deadline - _time.monotonic()
            if left <= 0:
                break
            try:
                r, st, val = q.get(timeout=min(left, 5.0))
            except _queue.Empty:
                if not any(p.is_alive() for p in procs) and q.empty():
                    break
                continue
            res[r] = (st, _unplain(val))
            if st != "ok":
                deadline = min(deadline, _time.monotonic() + grace)
    finally:
        for p in procs:
            p.join(grace)
        for p in procs:
            if p.is_alive() and nvls_off:
                p.kill()
                p.join(5)
    for r, (st, val) in sorted(res.items()):
        assert st == "ok", f"rank {r}: {val}"
    assert len(res) == world, f"only ranks {sorted(res)} of {world} reported"
    return res
