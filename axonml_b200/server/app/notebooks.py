"""Training notebooks of the platform server: documents of code/markdown cells, checkpoints, a
per-notebook Python kernel that executes code cells, and Jupyter ``.ipynb`` import/export.

Parity: cell types code/markdown, cell status idle/running/completed/error, notebook status
draft/running/completed/failed/stopped, ``CellOutput`` with output_type / text / execution_count /
error_name / error_value / traceback (crates/axonml-server/src/db/notebooks.rs:14-80); the
endpoints create / import / export / start / stop / add, update, delete and execute a cell
(api/notebooks.rs).  The reference's executor compiles Rust cells with cargo; here a cell is Python
run by a kernel process of the notebook (never inside the server process) in a namespace that
persists across the notebook's cells, with ``axonml_b200`` importable.  The AI-assist endpoint
asks the configured Ollama daemon (``integrations/ollama.py``) and answers 503 when none runs."""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import uuid

from .store import DocumentStore, NotFound, now_iso

CELL_TYPES = ("code", "markdown")


def new_cell(cell_type: str = "code", source: str = "") -> dict:
    if cell_type not in CELL_TYPES:
        raise ValueError(f"cell type must be one of {CELL_TYPES}")
    return {"id": uuid.uuid4().hex[:12], "cell_type": cell_type, "source": source, "outputs": [], "status": "idle",
            "execution_count": None, "metadata": {}}


# The kernel process: reads one JSON request per line on stdin ({"source": ...}), runs the cell in a
# namespace that lives as long as the process, and answers with one JSON line on the pipe it was
# started with.  Whatever the cell prints goes to buffers of this process only.
_WORKER = r"""
import ast, contextlib, io, json, os, sys, traceback
proto = os.fdopen(os.dup(1), "w")
devnull = os.open(os.devnull, os.O_WRONLY)
os.dup2(devnull, 1)
ns = {"__name__": "__notebook__"}
count = 0
for line in sys.stdin:
    req = json.loads(line)
    count += 1
    out, err = io.StringIO(), io.StringIO()
    outputs, ok = [], True
    try:
        tree = ast.parse(req["source"], mode="exec")
        last = None
        if tree.body and isinstance(tree.body[-1], ast.Expr):
            last = ast.Expression(tree.body.pop().value)
        with contextlib.redirect_stdout(out), contextlib.redirect_stderr(err):
            exec(compile(tree, "<cell>", "exec"), ns)
            value = eval(compile(last, "<cell>", "eval"), ns) if last is not None else None
        if out.getvalue():
            outputs.append({"output_type": "stream", "text": out.getvalue()})
        if err.getvalue():
            outputs.append({"output_type": "stream", "text": err.getvalue(), "data": {"name": "stderr"}})
        if value is not None:
            outputs.append({"output_type": "execute_result", "text": repr(value), "execution_count": count})
    except BaseException as e:
        ok = False
        if out.getvalue():
            outputs.append({"output_type": "stream", "text": out.getvalue()})
        outputs.append({"output_type": "error", "error_name": type(e).__name__, "error_value": str(e),
                        "traceback": traceback.format_exc().splitlines()})
    proto.write(json.dumps({"outputs": outputs, "ok": ok, "count": count}) + "\n")
    proto.flush()
"""


class NotebookKernel:
    """One Python process per notebook; cells run one at a time in a namespace that persists across
    the notebook's cells.  The process has its own working directory and a scrubbed environment
    (none of the server's secrets), and a cell that runs longer than ``timeout_s`` ends it: user
    code never runs inside the server process, which holds the token secret and every user's data
    (the reference likewise compiles and runs cells out of process)."""

    def __init__(self, timeout_s: float = 120.0, workdir: str | None = None):
        self.timeout_s = timeout_s
        self.count = 0
        self._lock = threading.Lock()
        self._own_dir = workdir is None
        self.workdir = workdir or tempfile.mkdtemp(prefix="axonml-nb-")
        self._proc: subprocess.Popen | None = None

    def _spawn(self) -> subprocess.Popen:
        env = {k: v for k, v in os.environ.items()
               if k in ("PATH", "HOME", "LANG", "LC_ALL", "LD_LIBRARY_PATH", "CUDA_VISIBLE_DEVICES", "VIRTUAL_ENV", "TMPDIR")}
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        env["PYTHONPATH"] = root
        return subprocess.Popen([sys.executable, "-u", "-c", _WORKER], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                stderr=subprocess.DEVNULL, cwd=self.workdir, env=env, text=True, bufsize=1)

    def _kill(self) -> None:
        p, self._proc = self._proc, None
        if p is not None:
            try:
                p.kill()          # the exact child this kernel started
                p.wait(5)
            except Exception:
                pass

    def close(self) -> None:
        with self._lock:
            self._kill()
            if self._own_dir:
                shutil.rmtree(self.workdir, ignore_errors=True)

    def __del__(self):
        try:
            self._kill()
        except Exception:
            pass

    def execute(self, source: str) -> tuple[list[dict], bool]:
        with self._lock:
            self.count += 1
            if self._proc is None or self._proc.poll() is not None:
                self._proc = self._spawn()
            p = self._proc
            answer: list = []

            def read():
                try:
                    answer.append(p.stdout.readline())
                except Exception:
                    answer.append("")
            try:
                p.stdin.write(json.dumps({"source": source}) + "\n")
                p.stdin.flush()
            except (BrokenPipeError, OSError):
                self._kill()
                return [_error_output("KernelDied", "the notebook kernel process is gone; it restarts on the next cell")], False
            t = threading.Thread(target=read, daemon=True)
            t.start()
            t.join(self.timeout_s)
            if t.is_alive():
                self._kill()
                return [_error_output("CellTimeout", f"the cell ran longer than {self.timeout_s:g} s; the kernel was restarted "
                                      "and its variables are gone")], False
            line = answer[0] if answer else ""
            if not line:
                self._kill()
                return [_error_output("KernelDied", "the notebook kernel process ended while running the cell")], False
            res = json.loads(line)
            for o in res["outputs"]:
                if "execution_count" in o:
                    o["execution_count"] = self.count
            return res["outputs"], bool(res["ok"])


def _error_output(name: str, value: str) -> dict:
    return {"output_type": "error", "error_name": name, "error_value": value, "traceback": []}


class NotebookService:
    def __init__(self, store: DocumentStore, cell_timeout_s: float = 120.0):
        self.col, self.ckpt = store["notebooks"], store["checkpoints"]
        self._kernels: dict[str, NotebookKernel] = {}
        self.cell_timeout_s = cell_timeout_s

    def _drop_kernel(self, nb_id: str) -> None:
        k = self._kernels.pop(nb_id, None)
        if k is not None:
            k.close()

    def shutdown(self) -> None:
        for nb_id in list(self._kernels):
            self._drop_kernel(nb_id)

    # ------------------------------------------------------------------ documents
    def create(self, user_id: str, name: str, description: str = "", cells: list[dict] | None = None) -> dict:
        return self.col.insert({"user_id": user_id, "name": name, "description": description, "status": "draft",
                                "cells": cells or [new_cell("markdown", f"# {name}"), new_cell("code", "")],
                                "metadata": {"kernel": "python", "framework": "axonml_b200"}})

    def get(self, nb_id: str) -> dict:
        return self.col.get(nb_id)

    def list(self, user_id: str | None = None) -> list[dict]:
        return self.col.find({"user_id": user_id} if user_id else None, sort="created_at", descending=True)

    def update(self, nb_id: str, **changes) -> dict:
        return self.col.update(nb_id, {k: v for k, v in changes.items() if k in ("name", "description", "cells", "metadata")})

    def delete(self, nb_id: str) -> None:
        self._drop_kernel(nb_id)
        self.ckpt.delete_where({"notebook_id": nb_id})
        self.col.delete(nb_id)

    # ------------------------------------------------------------------ cells
    def _cell_index(self, nb: dict, cell_id: str) -> int:
        for i, c in enumerate(nb["cells"]):
            if c["id"] == cell_id:
                return i
        raise NotFound(f"cell {cell_id}")

    def add_cell(self, nb_id: str, cell_type: str = "code", source: str = "", position: int | None = None) -> dict:
        nb = self.col.get(nb_id)
        c = new_cell(cell_type, source)
        nb["cells"].insert(len(nb["cells"]) if position is None else max(0, min(position, len(nb["cells"]))), c)
        self.col.update(nb_id, {"cells": nb["cells"]})
        return c

    def update_cell(self, nb_id: str, cell_id: str, source: str | None = None, cell_type: str | None = None) -> dict:
        nb = self.col.get(nb_id)
        i = self._cell_index(nb, cell_id)
        if source is not None:
            nb["cells"][i]["source"] = source
        if cell_type is not None:
            if cell_type not in CELL_TYPES:
                raise ValueError(f"cell type must be one of {CELL_TYPES}")
            nb["cells"][i]["cell_type"] = cell_type
        self.col.update(nb_id, {"cells": nb["cells"]})
        return nb["cells"][i]

    def delete_cell(self, nb_id: str, cell_id: str) -> None:
        nb = self.col.get(nb_id)
        del nb["cells"][self._cell_index(nb, cell_id)]
        self.col.update(nb_id, {"cells": nb["cells"]})

    # ------------------------------------------------------------------ execution
    def start(self, nb_id: str) -> dict:
        self._drop_kernel(nb_id)
        self._kernels[nb_id] = NotebookKernel(self.cell_timeout_s)
        return self.col.update(nb_id, {"status": "running"})

    def stop(self, nb_id: str) -> dict:
        self._drop_kernel(nb_id)
        return self.col.update(nb_id, {"status": "stopped"})

    def execute_cell(self, nb_id: str, cell_id: str) -> dict:
        nb = self.col.get(nb_id)
        i = self._cell_index(nb, cell_id)
        cell = nb["cells"][i]
        if cell["cell_type"] != "code":
            return cell
        k = self._kernels.get(nb_id)
        if k is None:
            k = self._kernels[nb_id] = NotebookKernel(self.cell_timeout_s)
        outputs, ok = k.execute(cell["source"])
        cell.update({"outputs": outputs, "status": "completed" if ok else "error", "execution_count": k.count})
        nb = self.col.get(nb_id)                     # other cells may have been edited while this one ran
        nb["cells"][self._cell_index(nb, cell_id)] = cell
        self.col.update(nb_id, {"cells": nb["cells"], "status": "running" if ok else "failed"})
        return cell

    def run_all(self, nb_id: str) -> dict:
        self.start(nb_id)
        ok = True
        for c in self.col.get(nb_id)["cells"]:
            if c["cell_type"] == "code" and c["source"].strip():
                ok = self.execute_cell(nb_id, c["id"])["status"] == "completed"
                if not ok:
                    break
        return self.col.update(nb_id, {"status": "completed" if ok else "failed"})

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, nb_id: str, label: str = "") -> dict:
        nb = self.col.get(nb_id)
        return self.ckpt.insert({"notebook_id": nb_id, "label": label, "cells": nb["cells"], "saved_at": now_iso()})

    def list_checkpoints(self, nb_id: str) -> list[dict]:
        return self.ckpt.find({"notebook_id": nb_id}, sort="created_at")

    def restore_checkpoint(self, nb_id: str, checkpoint_id: str) -> dict:
        ck = self.ckpt.get(checkpoint_id)
        if ck["notebook_id"] != nb_id:
            raise NotFound(f"checkpoint {checkpoint_id}")
        return self.col.update(nb_id, {"cells": ck["cells"]})

    # ------------------------------------------------------------------ ipynb
    def export_ipynb(self, nb_id: str) -> dict:
        nb = self.col.get(nb_id)
        cells = []
        for c in nb["cells"]:
            d = {"cell_type": c["cell_type"], "metadata": c.get("metadata", {}), "source": c["source"].splitlines(True)}
            if c["cell_type"] == "code":
                d["execution_count"] = c.get("execution_count")
                d["outputs"] = [_to_ipynb_output(o) for o in c.get("outputs", [])]
            cells.append(d)
        return {"nbformat": 4, "nbformat_minor": 5, "cells": cells,
                "metadata": {"kernelspec": {"name": "python3", "display_name": "Python 3", "language": "python"},
                             "axonml": {"name": nb["name"], "description": nb.get("description", "")}}}

    def import_ipynb(self, user_id: str, doc: dict | str, name: str | None = None) -> dict:
        if isinstance(doc, str):
            doc = json.loads(doc)
        cells = []
        for c in doc.get("cells", []):
            src = c.get("source", "")
            cell = new_cell("code" if c.get("cell_type") == "code" else "markdown", "".join(src) if isinstance(src, list) else src)
            cells.append(cell)
        meta = doc.get("metadata", {}).get("axonml", {})
        return self.create(user_id, name or meta.get("name") or "imported notebook", meta.get("description", ""), cells)


def _to_ipynb_output(o: dict) -> dict:
    t = o.get("output_type")
    if t == "stream":
        return {"output_type": "stream", "name": (o.get("data") or {}).get("name", "stdout"), "text": o.get("text", "")}
    if t == "error":
        return {"output_type": "error", "ename": o.get("error_name", ""), "evalue": o.get("error_value", ""),
                "traceback": o.get("traceback", [])}
    return {"output_type": "execute_result", "execution_count": o.get("execution_count"), "metadata": {},
            "data": {"text/plain": o.get("text", "")}}
