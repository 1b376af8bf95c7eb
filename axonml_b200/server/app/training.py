"""Training runs of the platform server: run records, a metrics tracker that fans new points out
to live subscribers, and an executor that runs the training on a worker thread.

Parity: run documents with status pending/running/completed/failed/stopped and a ``RunConfig`` of
epochs, batch_size, learning_rate, steps_per_epoch, optimizer (crates/axonml-server/src/db/runs.rs:17-100);
``TrainingTracker`` start/record/complete/stop/subscribe (training/tracker.rs:28-131); the stream
messages ``{"type": "metrics"|"status", "data": …}`` (training/websocket.rs:14-52).  The reference
executor fabricates a decaying loss curve (training/executor.rs:151-191); here the executor trains a
real model (MLP / SimpleCNN / LeNet on the configured or synthetic dataset) with this framework's
optimizers and reports the measured loss and accuracy."""
from __future__ import annotations

import queue
import threading
import time
import uuid

from .store import DocumentStore, NotFound, now_iso

RUN_STATUSES = ("pending", "running", "completed", "failed", "stopped")


def default_run_config(cfg: dict | None) -> dict:
    c = {"epochs": 1, "batch_size": 32, "learning_rate": 1e-3, "steps_per_epoch": 100, "optimizer": "adam"}
    c.update(cfg or {})
    return c


class RunRepository:
    def __init__(self, store: DocumentStore):
        self.runs, self.metrics, self.logs = store["runs"], store["metrics"], store["logs"]

    def create(self, user_id: str, name: str, model_type: str, config: dict | None = None, model_version_id=None,
               dataset_id=None) -> dict:
        return self.runs.insert({"user_id": user_id, "name": name, "model_type": model_type,
                                 "model_version_id": model_version_id, "dataset_id": dataset_id, "status": "pending",
                                 "config": default_run_config(config), "latest_metrics": None, "started_at": now_iso(),
                                 "completed_at": None})

    def get(self, run_id: str) -> dict:
        return self.runs.get(run_id)

    def list(self, user_id: str | None = None, status: str | None = None, limit=None, offset=0) -> list[dict]:
        flt = {}
        if user_id:
            flt["user_id"] = user_id
        if status:
            flt["status"] = status
        return self.runs.find(flt, limit=limit, offset=offset, sort="created_at", descending=True)

    def update_status(self, run_id: str, status: str) -> dict:
        if status not in RUN_STATUSES:
            raise ValueError(f"unknown run status {status!r}")
        ch = {"status": status}
        if status in ("completed", "failed", "stopped"):
            ch["completed_at"] = now_iso()
        return self.runs.update(run_id, ch)

    def record_metrics(self, run_id: str, m: dict) -> dict:
        m = dict(m)
        m.setdefault("timestamp", now_iso())
        m["run_id"] = run_id
        self.metrics.insert(m)
        self.runs.update(run_id, {"latest_metrics": {k: v for k, v in m.items() if k not in ("run_id", "id")}})
        return m

    def metrics_history(self, run_id: str, start_step: int | None = None, end_step: int | None = None, limit=None):
        flt: dict = {"run_id": run_id}
        if start_step is not None or end_step is not None:
            rng = {}
            if start_step is not None:
                rng["$gte"] = start_step
            if end_step is not None:
                rng["$lte"] = end_step
            flt["step"] = rng
        return self.metrics.find(flt, limit=limit, sort="step")

    def append_log(self, run_id: str, level: str, message: str) -> dict:
        return self.logs.insert({"run_id": run_id, "level": level, "message": message, "timestamp": now_iso()})

    def get_logs(self, run_id: str, limit: int | None = None) -> list[dict]:
        return self.logs.find({"run_id": run_id}, limit=limit, sort="created_at")

    def delete(self, run_id: str) -> None:
        self.runs.delete(run_id)
        self.metrics.delete_where({"run_id": run_id})
        self.logs.delete_where({"run_id": run_id})

    def count_running(self) -> int:
        return self.runs.count({"status": "running"})


class Subscription:
    """Receiving end of one live stream (a bounded queue: a slow reader loses old points, never
    blocks the trainer)."""

    def __init__(self, tracker: "TrainingTracker", run_id: str, maxsize: int = 1000):
        self.tracker, self.run_id, self.q = tracker, run_id, queue.Queue(maxsize)

    def push(self, msg: dict) -> None:
        try:
            self.q.put_nowait(msg)
        except queue.Full:
            try:
                self.q.get_nowait()
            except queue.Empty:
                pass
            self.q.put_nowait(msg)

    def get(self, timeout: float | None = None) -> dict | None:
        try:
            return self.q.get(timeout=timeout)
        except queue.Empty:
            return None

    def close(self) -> None:
        self.tracker.unsubscribe(self)


class TrainingTracker:
    def __init__(self, repo: RunRepository):
        self.repo = repo
        self._subs: dict[str, list[Subscription]] = {}
        self._active: set[str] = set()
        self._lock = threading.Lock()

    def start_run(self, run_id: str) -> None:
        self.repo.update_status(run_id, "running")
        with self._lock:
            self._active.add(run_id)
        self._broadcast(run_id, {"type": "status", "data": {"status": "running"}})

    def record_metrics(self, run_id: str, epoch: int, step: int, loss=None, accuracy=None, lr=None, gpu_util=None,
                       memory_mb=None, custom: dict | None = None) -> dict:
        m = {"epoch": epoch, "step": step, "loss": loss, "accuracy": accuracy, "lr": lr, "gpu_util": gpu_util,
             "memory_mb": memory_mb, "custom": custom or {}}
        m = self.repo.record_metrics(run_id, {k: v for k, v in m.items() if v is not None})
        self._broadcast(run_id, {"type": "metrics", "data": {k: v for k, v in m.items() if k not in ("run_id", "id")}})
        return m

    def complete_run(self, run_id: str, success: bool = True) -> None:
        self._finish(run_id, "completed" if success else "failed")

    def stop_run(self, run_id: str) -> None:
        self._finish(run_id, "stopped")

    def _finish(self, run_id: str, status: str) -> None:
        r = self.repo.update_status(run_id, status)
        with self._lock:
            self._active.discard(run_id)
        self._broadcast(run_id, {"type": "status", "data": {"status": status, "completed_at": r.get("completed_at")}})

    def is_tracking(self, run_id: str) -> bool:
        with self._lock:
            return run_id in self._active

    def subscribe(self, run_id: str) -> Subscription:
        s = Subscription(self, run_id)
        with self._lock:
            self._subs.setdefault(run_id, []).append(s)
        return s

    def unsubscribe(self, s: Subscription) -> None:
        with self._lock:
            if s in self._subs.get(s.run_id, []):
                self._subs[s.run_id].remove(s)

    def _broadcast(self, run_id: str, msg: dict) -> None:
        with self._lock:
            subs = list(self._subs.get(run_id, []))
        for s in subs:
            s.push(msg)


class TrainingExecutor:
    """Runs each training job on its own thread; ``stop(run_id)`` asks the loop to end after the
    current step."""

    def __init__(self, tracker: TrainingTracker, model_dir: str | None = None):
        self.tracker, self.model_dir = tracker, model_dir
        self._threads: dict[str, threading.Thread] = {}
        self._stops: dict[str, threading.Event] = {}

    def start(self, run: dict) -> None:
        ev = threading.Event()
        th = threading.Thread(target=self._run, args=(run, ev), daemon=True, name=f"train-{run['id'][:8]}")
        self._stops[run["id"]], self._threads[run["id"]] = ev, th
        th.start()

    def stop(self, run_id: str) -> bool:
        ev = self._stops.get(run_id)
        if ev is None:
            return False
        ev.set()
        return True

    def join(self, run_id: str, timeout: float | None = None) -> None:
        th = self._threads.get(run_id)
        if th is not None:
            th.join(timeout)

    def running(self) -> list[str]:
        return [r for r, t in self._threads.items() if t.is_alive()]

    # ------------------------------------------------------------------ the job
    def _run(self, run: dict, stop: threading.Event) -> None:
        rid, repo = run["id"], self.tracker.repo
        try:
            import torch
            from ... import nn
            from ...cli.config import ProjectConfig
            from ...cli.main import build_datasets, build_model, build_optimizer
            from ...data import DataLoader
            c = run["config"]
            cfg = ProjectConfig()
            cfg.model.architecture = {"mlp": "mlp", "cnn": "simplecnn", "simplecnn": "simplecnn",
                                      "lenet": "lenet"}.get(str(run.get("model_type", "mlp")).lower(), "mlp")
            cfg.training.epochs, cfg.training.batch_size = int(c["epochs"]), int(c["batch_size"])
            cfg.training.learning_rate = float(c["learning_rate"])
            cfg.training.optimizer.name = (c.get("optimizer") or "adam").lower()
            cfg.data.format = c.get("dataset_format", "synthetic-mnist")
            if c.get("dataset_path"):
                cfg.data.train_path = c["dataset_path"]
            dev = torch.device(c.get("device") or ("cuda" if torch.cuda.is_available() else "cpu"))
            torch.manual_seed(int(c.get("seed", 0)))
            model = build_model(cfg).to(dev)
            opt = build_optimizer(cfg, list(model.parameters()))
            train_ds, val_ds = build_datasets(cfg)
            loader = DataLoader(train_ds, cfg.training.batch_size, shuffle=True)
            crit = nn.CrossEntropyLoss()
            self.tracker.start_run(rid)
            repo.append_log(rid, "info", f"training {cfg.model.architecture} on {dev} ({train_ds.len()} samples)")
            step, limit = 0, int(c.get("steps_per_epoch", 0)) or None
            log_every = max(1, int(c.get("log_every", 10)))
            for epoch in range(cfg.training.epochs):
                hit = tot = 0
                for i, b in enumerate(loader):
                    if stop.is_set() or (limit is not None and i >= limit):
                        break
                    x, y = b.data.to(dev), b.targets.to(dev)
                    opt.zero_grad()
                    out = model(x)
                    loss = crit(out, y)
                    loss.backward()
                    opt.step()
                    step += 1
                    hit += int((out.detach().argmax(-1) == y).sum())
                    tot += y.numel()
                    if step % log_every == 0:
                        mem = torch.cuda.memory_allocated(dev) / 2 ** 20 if dev.type == "cuda" else None
                        self.tracker.record_metrics(rid, epoch + 1, step, float(loss.detach()), hit / max(tot, 1),
                                                    cfg.training.learning_rate, memory_mb=mem)
                if stop.is_set():
                    repo.append_log(rid, "warn", f"stopped at epoch {epoch + 1}, step {step}")
                    self.tracker.stop_run(rid)
                    return
                repo.append_log(rid, "info", f"epoch {epoch + 1} done: train accuracy {hit / max(tot, 1):.4f}")
            if self.model_dir:
                import os
                from ...serialize import save_state_dict
                from ...serialize.state_dict import StateDict
                os.makedirs(self.model_dir, exist_ok=True)
                path = os.path.join(self.model_dir, f"run_{rid}.axonml")
                save_state_dict(StateDict.from_module(model), path)
                repo.runs.update(rid, {"artifact": path})
            self.tracker.complete_run(rid, True)
        except Exception as e:  # noqa: BLE001 - the failure belongs in the run's log
            try:
                repo.append_log(rid, "error", f"{type(e).__name__}: {e}")
                self.tracker.complete_run(rid, False)
            except NotFound:
                pass


def new_id() -> str:
    return uuid.uuid4().hex
