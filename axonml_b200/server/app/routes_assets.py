"""Model, dataset, inference, hub and Kaggle routes (crates/axonml-server/src/api/{models,datasets,
data,inference,hub,kaggle,metrics}.rs; route table api/mod.rs:165-293)."""
from __future__ import annotations

import os
import time

from .api import PUBLIC, USER, HttpError


def register(app) -> None:
    r = app.router

    def _own(doc: dict, req) -> dict:
        if doc.get("user_id") not in (req.user_id, None) and req.claims.role != "admin":
            raise HttpError(403, "this item belongs to another user")
        return doc

    # ------------------------------------------------------------------ models
    def list_models(req):
        return app.registry.list_models(req.user_id if req.claims and req.claims.role != "admin" else None)

    def public_models(req):
        return [{k: m.get(k) for k in ("id", "name", "description", "model_type", "latest_version")}
                for m in app.registry.list_models()]

    def create_model(req):
        (name,) = req.need("name")
        return 201, app.registry.create_model(req.user_id, name, req.json.get("description", ""),
                                              req.json.get("model_type", "custom"))

    def get_model(req):
        return _own(app.registry.get_model(req.params["id"]), req)

    def update_model(req):
        _own(app.registry.get_model(req.params["id"]), req)
        return app.registry.update_model(req.params["id"], **req.json)

    def delete_model(req):
        _own(app.registry.get_model(req.params["id"]), req)
        app.registry.delete_model(req.params["id"])
        return {"deleted": True}

    def list_versions(req):
        _own(app.registry.get_model(req.params["id"]), req)
        return app.registry.list_versions(req.params["id"])

    def upload_version(req):
        _own(app.registry.get_model(req.params["id"]), req)
        fname, data, fields = req.upload()
        if not data:
            raise HttpError(400, "empty upload")
        return 201, app.registry.upload_version(req.params["id"], fname, data, fields.get("metrics") if isinstance(
            fields.get("metrics"), dict) else None, fields.get("training_run_id"))

    def get_version(req):
        _own(app.registry.get_model(req.params["id"]), req)
        return app.registry.get_version(req.params["id"], int(req.params["version"]))

    def delete_version(req):
        _own(app.registry.get_model(req.params["id"]), req)
        app.registry.delete_version(req.params["id"], int(req.params["version"]))
        return {"deleted": True}

    def download_version(req):
        _own(app.registry.get_model(req.params["id"]), req)
        return 200, (app.registry.read_version(req.params["id"], int(req.params["version"])), "application/octet-stream")

    def deploy_version(req):
        _own(app.registry.get_model(req.params["id"]), req)
        return app.registry.deploy_version(req.params["id"], int(req.params["version"]))

    r.add("GET", "/api/models", list_models)
    r.add("GET", "/api/public/models", public_models, PUBLIC)
    r.add("POST", "/api/models", create_model)
    r.add("GET", "/api/models/:id", get_model)
    r.add("PUT", "/api/models/:id", update_model)
    r.add("DELETE", "/api/models/:id", delete_model)
    r.add("GET", "/api/models/:id/versions", list_versions)
    r.add("POST", "/api/models/:id/versions", upload_version)
    r.add("GET", "/api/models/:id/versions/:version", get_version)
    r.add("DELETE", "/api/models/:id/versions/:version", delete_version)
    r.add("GET", "/api/models/:id/versions/:version/download", download_version)
    r.add("POST", "/api/models/:id/versions/:version/deploy", deploy_version)

    # ------------------------------------------------------------------ datasets + analysis
    def list_datasets(req):
        return app.datasets.list(req.user_id if req.claims.role != "admin" else None)

    def upload_dataset(req):
        fname, data, fields = req.upload()
        name = fields.get("name") or os.path.splitext(fname)[0]
        return 201, app.datasets.upload(req.user_id, name, fname, data, fields.get("dataset_type", "tabular"),
                                        fields.get("description", ""))

    def get_dataset(req):
        return _own(app.datasets.get(req.params["id"]), req)

    def delete_dataset(req):
        _own(app.datasets.get(req.params["id"]), req)
        app.datasets.delete(req.params["id"])
        return {"deleted": True}

    def _ds_path(req) -> str:
        return _own(app.datasets.get(req.params["id"]), req)["file_path"]

    def data_analyze(req):
        from ...data.analysis import analyze_dataset
        a = analyze_dataset(_ds_path(req), req.json.get("dataset_type"), int(req.json.get("max_samples", 10_000)))
        app.datasets.col.update(req.params["id"], {"num_samples": a.get("num_samples"), "num_features": a.get("num_features")})
        return a

    def data_preview(req):
        from ...data.analysis import preview_dataset
        return {"samples": preview_dataset(_ds_path(req), int(req.json.get("num_samples", 5)))}

    def data_validate(req):
        from ...data.analysis import validate_dataset
        return validate_dataset(_ds_path(req), req.json.get("num_classes"), req.json.get("input_shape"),
                                req.json.get("check_missing", True), req.json.get("check_balance", True))

    def data_generate_config(req):
        from ...data.analysis import generate_config
        fmt = req.json.get("format", "toml")
        return {"format": fmt, "config": generate_config(_ds_path(req), fmt)}

    def builtin_datasets(req):
        from ...data.catalog import BUILTIN_DATASETS
        return BUILTIN_DATASETS

    r.add("GET", "/api/datasets", list_datasets)
    r.add("POST", "/api/datasets", upload_dataset)
    r.add("GET", "/api/datasets/:id", get_dataset)
    r.add("DELETE", "/api/datasets/:id", delete_dataset)
    r.add("POST", "/api/data/:id/analyze", data_analyze)
    r.add("POST", "/api/data/:id/preview", data_preview)
    r.add("POST", "/api/data/:id/validate", data_validate)
    r.add("POST", "/api/data/:id/generate-config", data_generate_config)
    r.add("GET", "/api/builtin-datasets", builtin_datasets)

    # ------------------------------------------------------------------ inference
    def list_endpoints(req):
        return app.endpoints.list(req.user_id if req.claims.role != "admin" else None)

    def create_endpoint(req):
        name, model_id, version = req.need("name", "model_id", "version")
        _own(app.registry.get_model(model_id), req)
        return 201, app.endpoints.create(req.user_id, name, model_id, int(version), req.json.get("architecture"),
                                         int(req.json.get("replicas", 1)))

    def get_endpoint(req):
        return _own(app.endpoints.get(req.params["id"]), req)

    def delete_endpoint(req):
        _own(app.endpoints.get(req.params["id"]), req)
        app.endpoints.delete(req.params["id"])
        return {"deleted": True}

    def start_endpoint(req):
        _own(app.endpoints.get(req.params["id"]), req)
        return app.endpoints.start(req.params["id"])

    def stop_endpoint(req):
        _own(app.endpoints.get(req.params["id"]), req)
        return app.endpoints.stop(req.params["id"])

    def endpoint_metrics(req):
        e = _own(app.endpoints.get(req.params["id"]), req)
        return app.metrics.endpoint("/api/inference/predict/" + e["name"]).snapshot()

    def endpoint_info(req):
        e = _own(app.endpoints.get(req.params["id"]), req)
        m = app.inference.models.get(e["name"])
        info = {"endpoint": e, "loaded": m is not None}
        if m is not None:
            info["parameters"] = sum(p.numel() for p in m.parameters())
            info["device"] = str(app.inference.device)
        return info

    def predict(req):
        name = req.params["name"]
        t0 = time.perf_counter()
        try:
            out = app.inference.predict(name, req.need("input")[0])
        except KeyError:
            raise HttpError(404, f"no running endpoint named {name!r}") from None
        e = app.endpoints.col.find_one(name=name)
        if e is not None:
            app.endpoints.col.update(e["id"], {"request_count": int(e.get("request_count", 0)) + 1})
        return {"output": out, "latency_ms": (time.perf_counter() - t0) * 1e3}

    def completions(req):
        if app.engine is None:
            raise HttpError(404, "no language model is loaded")
        from ..http import AxonmlHTTPServer
        if not hasattr(app, "_llm_front"):
            front = AxonmlHTTPServer.__new__(AxonmlHTTPServer)      # reuse its engine thread + completion logic
            from ..http import _EngineThread
            front.engine, front.tokenizer = app.engine, app.tokenizer
            front._engine_thread = _EngineThread(app.engine)
            front._engine_thread.start()
            app._llm_front = front
        return app._llm_front.complete(req.json)

    def inference_status(req):
        return {"models_loaded": app.inference.list_models(), "endpoints_running": app.endpoints.count_running(),
                "llm": app.engine is not None, "device": str(app.inference.device)}

    def pool_status(req):
        p = app.inference.pool
        return {"entries": p.len(), "max_entries": p.max_entries, "idle_timeout_s": p.idle}

    def cache_status(req):
        from ... import hub
        d = hub.cache_dir()
        files = os.listdir(d) if os.path.isdir(d) else []
        return {"directory": d, "files": len(files), "bytes": sum(os.path.getsize(os.path.join(d, f)) for f in files)}

    def prometheus(req):
        extra = {"endpoints_running": app.endpoints.count_running(), "training_runs_running": app.runs.count_running(),
                 "users_total": app.users.count(), "uptime_seconds": time.time() - app.started}
        if app.engine is not None:
            s = app.engine.stats()
            extra.update({"llm_ttft_p50_seconds": s["ttft_p50_s"] or 0.0, "llm_decode_tokens_per_second": s["decode_tokens_per_s"],
                          "llm_queue_depth": s["queue_depth"], "llm_kv_page_occupancy": s["kv_page_occupancy"]})
        return 200, (app.metrics.prometheus(extra), "text/plain; version=0.0.4")

    r.add("GET", "/api/inference/endpoints", list_endpoints)
    r.add("POST", "/api/inference/endpoints", create_endpoint)
    r.add("GET", "/api/inference/endpoints/:id", get_endpoint)
    r.add("DELETE", "/api/inference/endpoints/:id", delete_endpoint)
    r.add("POST", "/api/inference/endpoints/:id/start", start_endpoint)
    r.add("POST", "/api/inference/endpoints/:id/stop", stop_endpoint)
    r.add("GET", "/api/inference/endpoints/:id/metrics", endpoint_metrics)
    r.add("GET", "/api/inference/endpoints/:id/info", endpoint_info)
    r.add("POST", "/api/inference/predict/:name", predict)
    r.add("POST", "/v1/completions", completions)
    r.add("GET", "/api/status/inference", inference_status, PUBLIC)
    r.add("GET", "/api/status/pool", pool_status, PUBLIC)
    r.add("GET", "/api/status/cache", cache_status, PUBLIC)
    r.add("GET", "/api/metrics", prometheus, PUBLIC)
    r.add("GET", "/metrics", prometheus, PUBLIC)

    # ------------------------------------------------------------------ hub
    def _hub_row(m) -> dict:
        from ... import hub
        return {"name": m.name, "architecture": m.architecture, "category": m.category.value, "parameters": m.num_parameters,
                "size_mb": round(m.size_mb(), 2), "description": m.description, "tasks": list(m.tasks),
                "cached": hub.is_cached(m.name)}

    def hub_list(req):
        from ... import hub
        q = req.q("q")
        return [_hub_row(m) for m in (hub.search_models(q) if q else hub.list_all_models())]

    def hub_info(req):
        from ... import hub
        m = hub.get_model_info(req.params["name"])
        if m is None:
            raise HttpError(404, f"unknown hub model {req.params['name']!r}")
        return _hub_row(m)

    def hub_download(req):
        """There is no weight server to download from: the model is built with fresh weights and
        written to the cache in the hub's weight format, so the load path is exercised."""
        from ... import hub
        m = hub.get_model_info(req.params["name"])
        if m is None:
            raise HttpError(404, f"unknown hub model {req.params['name']!r}")
        os.makedirs(hub.cache_dir(), exist_ok=True)
        path = os.path.join(hub.cache_dir(), m.name + ".weights")
        if not os.path.exists(path) or req.json.get("force"):
            model = m.build()
            hub.save_hub_weights({k: v.detach().cpu() for k, v in model.state_dict().items()}, path)
        return {"name": m.name, "path": path, "bytes": os.path.getsize(path), "source": "initialised locally"}

    def hub_cache(req):
        return cache_status(req)

    def hub_clear(req):
        from ... import hub
        d, n = hub.cache_dir(), 0
        name = req.params.get("name")
        for f in (os.listdir(d) if os.path.isdir(d) else []):
            if name is None or f == name + ".weights":
                os.remove(os.path.join(d, f))
                n += 1
        return {"removed": n}

    r.add("GET", "/api/hub/models", hub_list)
    r.add("GET", "/api/hub/models/:name", hub_info)
    r.add("POST", "/api/hub/models/:name/download", hub_download)
    r.add("GET", "/api/hub/cache", hub_cache)
    r.add("DELETE", "/api/hub/cache", hub_clear)
    r.add("DELETE", "/api/hub/cache/:name", hub_clear)

    # ------------------------------------------------------------------ kaggle
    def kaggle_save(req):
        from ...integrations.kaggle import KaggleClient
        username, key = req.need("username", "key")
        KaggleClient(config_dir=_kaggle_dir(app)).save_credentials(username, key)
        return {"configured": True}

    def kaggle_delete(req):
        from ...integrations.kaggle import KaggleClient
        KaggleClient(config_dir=_kaggle_dir(app)).delete_credentials()
        return {"configured": False}

    def kaggle_status(req):
        from ...integrations.kaggle import KaggleClient
        return KaggleClient(config_dir=_kaggle_dir(app)).status()

    def kaggle_search(req):
        from ...integrations.kaggle import KaggleClient, OfflineError
        try:
            return KaggleClient(config_dir=_kaggle_dir(app)).search(req.q("q", ""), req.q("limit", 10, int))
        except OfflineError as e:
            raise HttpError(503, str(e)) from None

    def kaggle_download(req):
        from ...integrations.kaggle import KaggleClient, OfflineError
        (ref,) = req.need("dataset")
        try:
            return KaggleClient(config_dir=_kaggle_dir(app)).download(ref, req.json.get("output_dir"))
        except OfflineError as e:
            raise HttpError(503, str(e)) from None

    def kaggle_downloaded(req):
        from ...integrations.kaggle import KaggleClient
        return KaggleClient(config_dir=_kaggle_dir(app)).list_downloaded()

    r.add("POST", "/api/kaggle/credentials", kaggle_save)
    r.add("DELETE", "/api/kaggle/credentials", kaggle_delete)
    r.add("GET", "/api/kaggle/status", kaggle_status)
    r.add("GET", "/api/kaggle/search", kaggle_search)
    r.add("POST", "/api/kaggle/download", kaggle_download)
    r.add("GET", "/api/kaggle/downloaded", kaggle_downloaded)
    _ = USER


def _kaggle_dir(app) -> str | None:
    return os.path.join(app.data_dir, "kaggle") if app.data_dir else None
