"""Model registry, dataset catalogue and inference endpoints of the platform server.

Parity: models with numbered versions whose files live under a storage directory, a deployable
version per endpoint (crates/axonml-server/src/api/models.rs, db/models.rs), uploaded datasets with
type/size/sample counts (api/datasets.rs), inference endpoints created/started/stopped against a
model version and served by the ``InferenceServer`` (api/inference.rs)."""
from __future__ import annotations

import hashlib
import os

from .store import AlreadyExists, DocumentStore, NotFound

_MODEL_EXTS = {".axonml": "axonml", ".safetensors": "safetensors", ".json": "json", ".onnx": "onnx", ".gguf": "gguf",
               ".pt": "pytorch", ".pth": "pytorch", ".bin": "binary"}


def detect_format(filename: str) -> str:
    return _MODEL_EXTS.get(os.path.splitext(filename)[1].lower(), "unknown")


class ModelRegistry:
    def __init__(self, store: DocumentStore, storage_dir: str):
        self.models, self.versions = store["models"], store["versions"]
        self.dir = storage_dir
        os.makedirs(storage_dir, exist_ok=True)

    # ------------------------------------------------------------------ models
    def create_model(self, user_id: str, name: str, description: str = "", model_type: str = "custom") -> dict:
        if self.models.find_one(user_id=user_id, name=name):
            raise AlreadyExists(f"model {name!r}")
        return self.models.insert({"user_id": user_id, "name": name, "description": description, "model_type": model_type,
                                   "version_count": 0, "latest_version": None})

    def get_model(self, model_id: str) -> dict:
        return self.models.get(model_id)

    def list_models(self, user_id: str | None = None) -> list[dict]:
        return self.models.find({"user_id": user_id} if user_id else None, sort="created_at", descending=True)

    def update_model(self, model_id: str, **changes) -> dict:
        return self.models.update(model_id, {k: v for k, v in changes.items() if k in ("name", "description", "model_type")})

    def delete_model(self, model_id: str) -> None:
        for v in self.list_versions(model_id):
            self.delete_version(model_id, v["version"])
        self.models.delete(model_id)

    # ------------------------------------------------------------------ versions
    def upload_version(self, model_id: str, filename: str, data: bytes, metrics: dict | None = None,
                       training_run_id: str | None = None) -> dict:
        m = self.models.get(model_id)
        version = int(m.get("version_count", 0)) + 1
        d = os.path.join(self.dir, model_id, f"v{version}")
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, os.path.basename(filename) or "model.axonml")
        with open(path, "wb") as f:
            f.write(data)
        doc = self.versions.insert({"model_id": model_id, "version": version, "file_path": path, "file_size": len(data),
                                    "format": detect_format(filename), "sha256": hashlib.sha256(data).hexdigest(),
                                    "metrics": metrics or {}, "training_run_id": training_run_id, "deployed": False})
        self.models.update(model_id, {"version_count": version, "latest_version": version})
        return doc

    def list_versions(self, model_id: str) -> list[dict]:
        return self.versions.find({"model_id": model_id}, sort="version")

    def get_version(self, model_id: str, version: int) -> dict:
        v = self.versions.find_one(model_id=model_id, version=int(version))
        if v is None:
            raise NotFound(f"model {model_id} version {version}")
        return v

    def read_version(self, model_id: str, version: int) -> bytes:
        with open(self.get_version(model_id, version)["file_path"], "rb") as f:
            return f.read()

    def delete_version(self, model_id: str, version: int) -> None:
        v = self.get_version(model_id, version)
        if os.path.exists(v["file_path"]):
            os.remove(v["file_path"])
        self.versions.delete(v["id"])

    def deploy_version(self, model_id: str, version: int) -> dict:
        for v in self.list_versions(model_id):
            if v["deployed"]:
                self.versions.update(v["id"], {"deployed": False})
        return self.versions.update(self.get_version(model_id, version)["id"], {"deployed": True})


class DatasetCatalog:
    def __init__(self, store: DocumentStore, storage_dir: str):
        self.col, self.dir = store["datasets"], storage_dir
        os.makedirs(storage_dir, exist_ok=True)

    def upload(self, user_id: str, name: str, filename: str, data: bytes, dataset_type: str = "tabular",
               description: str = "") -> dict:
        if self.col.find_one(user_id=user_id, name=name):
            raise AlreadyExists(f"dataset {name!r}")
        doc = self.col.insert({"user_id": user_id, "name": name, "description": description, "dataset_type": dataset_type,
                               "file_path": "", "file_size": len(data), "num_samples": None, "num_features": None})
        d = os.path.join(self.dir, doc["id"])
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, os.path.basename(filename) or "data.bin")
        with open(path, "wb") as f:
            f.write(data)
        info = {"file_path": path}
        if path.endswith(".csv"):
            text = data.decode("utf-8", "replace").splitlines()
            info["num_samples"] = max(len(text) - 1, 0)
            info["num_features"] = len(text[0].split(",")) if text else 0
        return self.col.update(doc["id"], info)

    def register_path(self, user_id: str, name: str, path: str, dataset_type: str = "image") -> dict:
        """A dataset that already lies on the server's disk (built-in or downloaded)."""
        size = sum(os.path.getsize(os.path.join(r, f)) for r, _, fs in os.walk(path) for f in fs) if os.path.isdir(path) \
            else os.path.getsize(path)
        return self.col.insert({"user_id": user_id, "name": name, "description": "", "dataset_type": dataset_type,
                                "file_path": path, "file_size": size, "num_samples": None, "num_features": None})

    def get(self, dataset_id: str) -> dict:
        return self.col.get(dataset_id)

    def list(self, user_id: str | None = None) -> list[dict]:
        return self.col.find({"user_id": user_id} if user_id else None, sort="created_at", descending=True)

    def delete(self, dataset_id: str) -> None:
        d = self.col.get(dataset_id)
        own = os.path.join(self.dir, dataset_id)
        if d["file_path"].startswith(own) and os.path.exists(d["file_path"]):
            os.remove(d["file_path"])
            os.rmdir(own)
        self.col.delete(dataset_id)


class EndpointManager:
    """Inference endpoints: a named route bound to a model version; ``start`` loads the weights into
    the ``InferenceServer`` (``/api/inference/predict/<name>`` then answers), ``stop`` unloads."""

    def __init__(self, store: DocumentStore, registry: ModelRegistry, inference):
        self.col, self.registry, self.inference = store["endpoints"], registry, inference

    def create(self, user_id: str, name: str, model_id: str, version: int, architecture: dict | None = None,
               replicas: int = 1) -> dict:
        if self.col.find_one(name=name):
            raise AlreadyExists(f"endpoint {name!r}")
        self.registry.get_version(model_id, version)
        return self.col.insert({"user_id": user_id, "name": name, "model_id": model_id, "version": int(version),
                                "architecture": architecture or {}, "replicas": replicas, "status": "stopped",
                                "request_count": 0, "error": None})

    def get(self, endpoint_id: str) -> dict:
        return self.col.get(endpoint_id)

    def list(self, user_id: str | None = None) -> list[dict]:
        return self.col.find({"user_id": user_id} if user_id else None, sort="created_at")

    def start(self, endpoint_id: str) -> dict:
        e = self.col.get(endpoint_id)
        v = self.registry.get_version(e["model_id"], e["version"])
        try:
            self.inference.load(e["name"], v["file_path"], (e.get("architecture") or {}).get("activation", "relu"))
            return self.col.update(endpoint_id, {"status": "running", "error": None})
        except Exception as ex:  # noqa: BLE001 - recorded on the endpoint
            return self.col.update(endpoint_id, {"status": "error", "error": f"{type(ex).__name__}: {ex}"})

    def stop(self, endpoint_id: str) -> dict:
        e = self.col.get(endpoint_id)
        self.inference.unload(e["name"])
        return self.col.update(endpoint_id, {"status": "stopped"})

    def delete(self, endpoint_id: str) -> None:
        e = self.col.get(endpoint_id)
        if e["status"] == "running":
            self.inference.unload(e["name"])
        self.col.delete(endpoint_id)

    def count_running(self) -> int:
        return self.col.count({"status": "running"})
