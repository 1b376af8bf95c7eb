"""Weights & Biases logging (crates/axonml-cli/src/commands/wandb.rs, wandb_client.rs:76-267): the
settings file (api key, entity, project, base URL, log frequency, enabled flag) and a run object
with ``log`` / ``log_at_step`` / ``summary`` / ``log_config`` / ``flush`` / ``finish``.

The run is always written in offline-run layout under ``<dir>/offline-run-<time>-<id>/`` —
``files/config.yaml``, ``files/wandb-summary.json``, ``files/wandb-history.jsonl`` and
``files/wandb-metadata.json`` — so a host with network access can upload it later; no request
leaves the process from here."""
from __future__ import annotations

import json
import os
import platform
import secrets
import time
from dataclasses import asdict, dataclass


def _settings_path() -> str:
    base = os.environ.get("AXONML_CONFIG_DIR") or os.path.join(os.path.expanduser("~"), ".config", "axonml")
    return os.path.join(base, "wandb.json")


@dataclass
class WandbConfig:
    api_key: str | None = None
    entity: str | None = None
    project: str = "axonml"
    base_url: str = "https://api.wandb.ai"
    log_frequency: int = 10
    log_checkpoints: bool = False
    log_system: bool = True
    enabled: bool = False

    @classmethod
    def load(cls, path: str | None = None) -> "WandbConfig":
        try:
            with open(path or _settings_path()) as f:
                d = json.load(f)
            return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})
        except (OSError, ValueError):
            c = cls()
            c.api_key = os.environ.get("WANDB_API_KEY")
            return c

    def save(self, path: str | None = None) -> str:
        p = path or _settings_path()
        os.makedirs(os.path.dirname(p), exist_ok=True)
        fd = os.open(p, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
        with os.fdopen(fd, "w") as f:
            json.dump(asdict(self), f, indent=1)
        return p

    def is_logged_in(self) -> bool:
        return bool(self.api_key)

    def status(self) -> dict:
        d = asdict(self)
        d["api_key"] = ("*" * 8 + self.api_key[-4:]) if self.api_key else None
        d["logged_in"] = self.is_logged_in()
        return d


class WandbRun:
    def __init__(self, project: str, name: str | None = None, entity: str | None = None, config: dict | None = None,
                 directory: str = "./wandb", log_frequency: int = 1):
        self.project, self.entity = project, entity or "offline"
        self.id = secrets.token_hex(4)
        self.name = name or f"run-{self.id}"
        self.dir = os.path.join(directory, f"offline-run-{time.strftime('%Y%m%d_%H%M%S')}-{self.id}")
        self.files = os.path.join(self.dir, "files")
        os.makedirs(self.files, exist_ok=True)
        self._step, self._buf, self._summary, self._every = 0, [], {}, max(1, log_frequency)
        self._t0 = time.time()
        self.log_config(config or {})
        with open(os.path.join(self.files, "wandb-metadata.json"), "w") as f:
            json.dump({"project": project, "entity": self.entity, "name": self.name, "id": self.id,
                       "host": platform.node(), "python": platform.python_version(), "startedAt": time.strftime(
                           "%Y-%m-%dT%H:%M:%S", time.gmtime()), "framework": "axonml_b200"}, f, indent=1)

    @classmethod
    def init(cls, project, name=None, entity=None, config=None, **kw) -> "WandbRun":
        return cls(project, name, entity, config, **kw)

    def url(self) -> str:
        return f"https://wandb.ai/{self.entity}/{self.project}/runs/{self.id}"

    def current_step(self) -> int:
        return self._step

    def log(self, metrics: dict) -> None:
        self.log_at_step(self._step, metrics)
        self._step += 1

    def log_at_step(self, step: int, metrics: dict) -> None:
        row = {k: float(v) for k, v in metrics.items()}
        row.update({"_step": int(step), "_runtime": time.time() - self._t0, "_timestamp": time.time()})
        self._buf.append(row)
        self._summary.update({k: v for k, v in row.items() if not k.startswith("_")})
        self._step = max(self._step, int(step))
        if len(self._buf) >= self._every:
            self.flush()

    def summary(self, key: str, value: float) -> None:
        self._summary[key] = float(value)

    def log_config(self, config: dict) -> None:
        import yaml
        path = os.path.join(self.files, "config.yaml")
        cur = {}
        if os.path.exists(path):
            with open(path) as f:
                cur = yaml.safe_load(f) or {}
        cur.update({k: {"value": v} for k, v in config.items()})
        with open(path, "w") as f:
            yaml.safe_dump(cur, f)

    def flush(self) -> None:
        if self._buf:
            with open(os.path.join(self.files, "wandb-history.jsonl"), "a") as f:
                for row in self._buf:
                    f.write(json.dumps(row) + "\n")
            self._buf = []
        with open(os.path.join(self.files, "wandb-summary.json"), "w") as f:
            json.dump(self._summary, f)

    def finish(self) -> str:
        self._summary["_runtime"] = time.time() - self._t0
        self.flush()
        return self.dir


def init_training_run(cfg: WandbConfig, run_name: str, hyper: dict, directory: str = "./wandb") -> WandbRun | None:
    """The hook ``train`` calls: a run when logging is enabled, else None."""
    if not cfg.enabled:
        return None
    return WandbRun(cfg.project, run_name, cfg.entity, hyper, directory, cfg.log_frequency)
