"""System, notebook, terminal and dashboard routes (crates/axonml-server/src/api/{system,notebooks,
terminal}.rs; route table api/mod.rs:222-230, 296-331, 381-382) and ``/health``."""
from __future__ import annotations

import os
import time

from . import websocket as WS
from .api import PUBLIC, USER, HttpError


def register(app) -> None:
    r = app.router

    def health(req):
        return {"status": "healthy", "uptime_s": time.time() - app.started, "database": app.store.health()["status"],
                "version": "axonml_b200"}

    r.add("GET", "/health", health, PUBLIC)

    # ------------------------------------------------------------------ system
    def sys_info(req):
        from .system import system_info
        return system_info()

    def sys_gpus(req):
        from .system import list_gpus
        return list_gpus()

    def sys_benchmark(req):
        from .system import run_benchmark
        return run_benchmark(int(req.json.get("size", 1024)), int(req.json.get("iterations", 5)), req.json.get("device"))

    r.add("GET", "/api/system/info", sys_info)
    r.add("GET", "/api/system/gpus", sys_gpus)
    r.add("POST", "/api/system/benchmark", sys_benchmark)
    r.add("GET", "/api/system/metrics", lambda req: app.monitor.sample())
    r.add("GET", "/api/system/metrics/history", lambda req: app.monitor.history())
    r.add("GET", "/api/system/correlation", lambda req: app.monitor.correlation())

    # ------------------------------------------------------------------ notebooks
    nb = app.notebooks

    def _own_nb(req) -> dict:
        d = nb.get(req.params["id"])
        if d["user_id"] != req.user_id and req.claims.role != "admin":
            raise HttpError(403, "this notebook belongs to another user")
        return d

    def nb_create(req):
        (name,) = req.need("name")
        return 201, nb.create(req.user_id, name, req.json.get("description", ""), req.json.get("cells"))

    def nb_import(req):
        doc = req.json.get("notebook") or req.json
        return 201, nb.import_ipynb(req.user_id, doc, req.json.get("name"))

    def nb_update(req):
        _own_nb(req)
        return nb.update(req.params["id"], **req.json)

    def nb_delete(req):
        _own_nb(req)
        nb.delete(req.params["id"])
        return {"deleted": True}

    def nb_add_cell(req):
        _own_nb(req)
        return 201, nb.add_cell(req.params["id"], req.json.get("cell_type", "code"), req.json.get("source", ""),
                                req.json.get("position"))

    def nb_update_cell(req):
        _own_nb(req)
        return nb.update_cell(req.params["id"], req.params["cell"], req.json.get("source"), req.json.get("cell_type"))

    def nb_delete_cell(req):
        _own_nb(req)
        nb.delete_cell(req.params["id"], req.params["cell"])
        return {"deleted": True}

    def _may_run_code(req) -> None:
        _own_nb(req)
        if req.claims.role not in ("admin", "user"):
            raise HttpError(403, "running notebook code needs the user or admin role")

    def nb_execute_cell(req):
        _may_run_code(req)
        return nb.execute_cell(req.params["id"], req.params["cell"])

    def nb_ai_assist(req):
        """A code or markdown suggestion for the notebook from the configured Ollama daemon; the
        notebook's existing cells are sent as context (api/notebooks.rs ai_assist)."""
        from ...integrations.ollama import DEFAULT_MODEL, DEFAULT_URL, OllamaClient, OllamaError
        doc = _own_nb(req)
        (prompt,) = req.need("prompt")
        client = OllamaClient(app.ollama_url or DEFAULT_URL, (req.json or {}).get("model") or app.ollama_model or DEFAULT_MODEL)
        if not client.is_available():
            raise HttpError(503, f"AI assist needs an Ollama daemon; none answers at {client.base_url}")
        context = "\n\n".join(f"[{c.get('cell_type', 'code')}]\n{c.get('source', '')}" for c in doc.get("cells", [])[-8:]) \
            if (req.json or {}).get("include_context", True) else ""
        try:
            if (req.json or {}).get("cell_type", "code") == "markdown":
                return client.generate_markdown(prompt, context)
            return client.generate_code(prompt, context)
        except OllamaError as e:
            raise HttpError(502, str(e)) from None

    def nb_restore(req):
        _own_nb(req)
        return nb.restore_checkpoint(req.params["id"], req.params["ckpt"])

    r.add("GET", "/api/notebooks", lambda req: nb.list(req.user_id if req.claims.role != "admin" else None))
    r.add("POST", "/api/notebooks", nb_create)
    r.add("POST", "/api/notebooks/import", nb_import)
    r.add("GET", "/api/notebooks/:id", lambda req: _own_nb(req))
    r.add("PUT", "/api/notebooks/:id", nb_update)
    r.add("DELETE", "/api/notebooks/:id", nb_delete)
    r.add("GET", "/api/notebooks/:id/export", lambda req: (_own_nb(req), nb.export_ipynb(req.params["id"]))[1])
    r.add("POST", "/api/notebooks/:id/start", lambda req: (_may_run_code(req), nb.start(req.params["id"]))[1])
    r.add("POST", "/api/notebooks/:id/stop", lambda req: (_own_nb(req), nb.stop(req.params["id"]))[1])
    r.add("POST", "/api/notebooks/:id/run-all", lambda req: (_may_run_code(req), nb.run_all(req.params["id"]))[1])
    r.add("POST", "/api/notebooks/:id/cells", nb_add_cell)
    r.add("PUT", "/api/notebooks/:id/cells/:cell", nb_update_cell)
    r.add("DELETE", "/api/notebooks/:id/cells/:cell", nb_delete_cell)
    r.add("POST", "/api/notebooks/:id/cells/:cell/execute", nb_execute_cell)
    r.add("POST", "/api/notebooks/:id/ai-assist", nb_ai_assist)
    r.add("GET", "/api/notebooks/:id/checkpoints", lambda req: (_own_nb(req), nb.list_checkpoints(req.params["id"]))[1])
    r.add("POST", "/api/notebooks/:id/checkpoints",
          lambda req: (_own_nb(req), (201, nb.save_checkpoint(req.params["id"], req.json.get("label", ""))))[1])
    r.add("POST", "/api/notebooks/:id/checkpoints/:ckpt/restore", nb_restore)

    # ------------------------------------------------------------------ terminal (PTY over WebSocket)
    def terminal_info(req):
        return {"enabled": app.enable_terminal, "shell": os.environ.get("SHELL", "/bin/sh"),
                "note": None if app.enable_terminal else "start the server with enable_terminal=True (administrators only)"}

    def terminal_ws(req):
        if not app.enable_terminal:
            raise HttpError(403, "the terminal is disabled on this server")
        if req.claims.role != "admin":
            raise HttpError(403, "administrator role required")
        ws = WS.upgrade(req.handler) if req.handler is not None else None
        if ws is None:
            raise HttpError(400, "this route is a WebSocket endpoint")
        _run_pty(ws, os.environ.get("SHELL", "/bin/sh"))
        return None

    r.add("GET", "/api/terminal/info", terminal_info)
    r.add("GET", "/api/terminal", terminal_ws)

    # ------------------------------------------------------------------ dashboard
    def dashboard(req):
        from .dashboard import PAGE
        return 200, (PAGE, "text/html; charset=utf-8")

    r.add("GET", "/", dashboard, PUBLIC)
    r.add("GET", "/dashboard", dashboard, PUBLIC)
    _ = USER


def _run_pty(ws, shell: str) -> None:
    """Bridges a WebSocket to a shell on a pseudo-terminal: text frames are keystrokes, JSON
    ``{"type": "resize", "cols": c, "rows": r}`` resizes, output goes back as text frames."""
    import fcntl
    import json
    import pty
    import select
    import struct
    import termios
    pid, fd = pty.fork()
    if pid == 0:
        os.execvp(shell, [shell])
    try:
        while not ws.closed:
            rd, _, _ = select.select([fd, ws.sock], [], [], 0.5)
            if fd in rd:
                try:
                    data = os.read(fd, 65536)
                except OSError:
                    break
                if not data:
                    break
                ws.send_text(data.decode("utf-8", "replace"))
            if ws.sock in rd:
                try:
                    msg = ws.recv(timeout=1.0)
                except WS.WebSocketClosed:
                    break
                if msg is None:
                    continue
                if isinstance(msg, str) and msg.startswith('{"type"'):
                    try:
                        j = json.loads(msg)
                        if j.get("type") == "resize":
                            fcntl.ioctl(fd, termios.TIOCSWINSZ, struct.pack("HHHH", int(j["rows"]), int(j["cols"]), 0, 0))
                            continue
                    except (ValueError, KeyError):
                        pass
                os.write(fd, msg.encode() if isinstance(msg, str) else msg)
    finally:
        try:
            os.close(fd)
        except OSError:
            pass
        try:
            os.kill(pid, 15)
            os.waitpid(pid, 0)
        except OSError:
            pass
        ws.close()
