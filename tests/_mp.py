"""Helper: run a function as N CPU ranks (gloo) in child processes and collect their results."""
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _plain(x):
    """Tensors cross the process boundary as numpy arrays (no shared file descriptors)."""
    if torch.is_tensor(x):
        return ("__t__", x.detach().cpu().float().numpy() if x.dtype == torch.bfloat16 else x.detach().cpu().numpy())
    if isinstance(x, dict):
        return {k: _plain(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_plain(v) for v in x)
    return x


def _unplain(x):
    if isinstance(x, tuple) and len(x) == 2 and isinstance(x[0], str) and x[0] == "__t__":
        return torch.from_numpy(x[1])
    if isinstance(x, dict):
        return {k: _unplain(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_unplain(v) for v in x)
    return x


def _entry(rank, world, port, fn, args, q, timeout_s):
    try:
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        torch.set_num_threads(1)
        from axonml_b200.parallel import CpuBackend
        be = CpuBackend.init(rank, world, "127.0.0.1", port, timeout_s=timeout_s)
        out = fn(rank, world, be, *args)
        q.put((rank, "ok", _plain(out)))
        try:
            be.destroy()
        except Exception:
            pass
    except Exception as e:  # noqa: BLE001
        q.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


def run_ranks(fn, world: int = 2, args=(), timeout_s: float = 60.0, expect_all_ok: bool = True,
              skip_ranks=()):
    """Spawns ``world`` ranks (minus ``skip_ranks``, which never join).  Returns {rank: (status,
    value)}."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = []
    for r in range(world):
        if r in skip_ranks:
            continue
        p = ctx.Process(target=_entry, args=(r, world, port, fn, args, q, timeout_s), daemon=True)
        p.start()
        procs.append(p)
    res = {}
    for _ in procs:
        r, st, val = q.get(timeout=timeout_s + 120)
        res[r] = (st, _unplain(val))
    for p in procs:
        p.join(30)
        if p.is_alive():
            p.kill()
    if expect_all_ok:
        for r, (st, val) in res.items():
            assert st == "ok", f"rank {r}: {val}"
    return res
