"""Training-run routes (crates/axonml-server/src/api/training.rs; route table api/mod.rs:148-163):
list / create / get / delete / stop a run, metrics history, logs, and the live WebSocket stream of
``{"type": "metrics"|"status", "data": …}`` messages (training/websocket.rs)."""
from __future__ import annotations

from . import websocket as WS
from .api import USER, HttpError


def register(app) -> None:
    r = app.router

    def _own_run(req) -> dict:
        run = app.runs.get(req.params["id"])
        if run["user_id"] != req.user_id and req.claims.role != "admin":
            raise HttpError(403, "this run belongs to another user")
        return run

    def list_runs(req):
        uid = None if (req.claims.role == "admin" and req.q("all")) else req.user_id
        return app.runs.list(uid, req.q("status"), req.q("limit", None, int), req.q("offset", 0, int))

    def create_run(req):
        name, model_type = req.need("name", "model_type")
        run = app.runs.create(req.user_id, name, model_type, req.json.get("config"), req.json.get("model_version_id"),
                              req.json.get("dataset_id"))
        ds_id = req.json.get("dataset_id")
        if ds_id:
            ds = app.datasets.get(ds_id)
            run["config"].setdefault("dataset_path", ds["file_path"])
        if req.json.get("start", True):
            app.executor.start(run)
        return 201, run

    def get_run(req):
        return _own_run(req)

    def delete_run(req):
        run = _own_run(req)
        app.executor.stop(run["id"])
        app.executor.join(run["id"], 5.0)
        app.runs.delete(run["id"])
        return {"deleted": True}

    def stop_run(req):
        run = _own_run(req)
        if not app.executor.stop(run["id"]) and run["status"] in ("pending", "running"):
            app.tracker.stop_run(run["id"])          # a run recorded by an external trainer
        return {"stopping": True}

    def complete_run(req):
        run = _own_run(req)
        app.tracker.complete_run(run["id"], bool(req.json.get("success", True)))
        return app.runs.get(run["id"])

    def get_metrics(req):
        run = _own_run(req)
        return app.runs.metrics_history(run["id"], req.q("start_step", None, int), req.q("end_step", None, int),
                                        req.q("limit", None, int))

    def post_metrics(req):
        """An external trainer (the CLI's ``train --sync``) reports a point."""
        run = _own_run(req)
        if run["status"] == "pending":
            app.tracker.start_run(run["id"])
        j = req.json
        return app.tracker.record_metrics(run["id"], int(j.get("epoch", 0)), int(j.get("step", 0)), j.get("loss"),
                                          j.get("accuracy"), j.get("lr"), j.get("gpu_util"), j.get("memory_mb"),
                                          j.get("custom"))

    def get_logs(req):
        return app.runs.get_logs(_own_run(req)["id"], req.q("limit", None, int))

    def append_log(req):
        run = _own_run(req)
        (message,) = req.need("message")
        return 201, app.runs.append_log(run["id"], req.json.get("level", "info"), message)

    def stream(req):
        run = _own_run(req)
        ws = WS.upgrade(req.handler) if req.handler is not None else None
        if ws is None:
            raise HttpError(400, "this route is a WebSocket endpoint")
        sub = app.tracker.subscribe(run["id"])
        try:
            ws.send_json({"type": "status", "data": {"status": app.runs.get(run["id"])["status"]}})
            while not ws.closed:
                msg = sub.get(timeout=0.25)
                if msg is not None:
                    ws.send_json(msg)
                    if msg["type"] == "status" and msg["data"]["status"] in ("completed", "failed", "stopped"):
                        break
                else:
                    try:
                        ws.recv(timeout=0.001)       # notices a client that went away
                    except WS.WebSocketClosed:
                        break
        except WS.WebSocketClosed:
            pass
        finally:
            sub.close()
            ws.close()
        return None

    r.add("GET", "/api/training/runs", list_runs)
    r.add("POST", "/api/training/runs", create_run)
    r.add("GET", "/api/training/runs/:id", get_run)
    r.add("DELETE", "/api/training/runs/:id", delete_run)
    r.add("POST", "/api/training/runs/:id/stop", stop_run)
    r.add("POST", "/api/training/runs/:id/complete", complete_run)
    r.add("GET", "/api/training/runs/:id/metrics", get_metrics)
    r.add("POST", "/api/training/runs/:id/metrics", post_metrics)
    r.add("GET", "/api/training/runs/:id/stream", stream)
    r.add("GET", "/api/training/runs/:id/logs", get_logs)
    r.add("POST", "/api/training/runs/:id/logs", append_log)
    _ = USER
