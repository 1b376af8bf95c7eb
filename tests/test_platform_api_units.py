"""The platform server's REST API route by route over a real socket: who may call what, what a
missing record answers, and the small lifecycles (the topics of the reference's integration tests
under crates/axonml-server/tests: api_auth, api_models, api_inference, api_training, api_admin,
api_system, api_datasets, api_hub, error handling, concurrent requests).  CPU only."""
import concurrent.futures as cf
import json
import time
import urllib.request

import pytest

from axonml_b200.server.app import PlatformServer
from tests.test_platform_server import Client

ADMIN = {"email": "admin@example.com", "name": "Admin", "password": "s3cret-pass"}


@pytest.fixture(scope="module")
def srv(tmp_path_factory):
    s = PlatformServer(port=0, data_dir=str(tmp_path_factory.mktemp("platform"))).start()
    c = Client(s.port)
    st, j = c.req("POST", "/api/auth/register", ADMIN)
    assert st == 201, j
    yield s
    s.stop()


@pytest.fixture()
def anon(srv):
    return Client(srv.port)


@pytest.fixture()
def admin(srv):
    c = Client(srv.port)
    st, j = c.req("POST", "/api/auth/login", {"email": ADMIN["email"], "password": ADMIN["password"]})
    assert st == 200, j
    c.token = j["access_token"]
    c.refresh = j["refresh_token"]
    return c


# ------------------------------------------------------------------------------------------ auth
def test_health_endpoint(anon):
    st, j = anon.req("GET", "/health")
    assert st == 200 and j["status"] == "healthy"


def test_login_with_valid_credentials(anon):
    st, j = anon.req("POST", "/api/auth/login", {"email": ADMIN["email"], "password": ADMIN["password"]})
    assert st == 200 and j["access_token"] and j["refresh_token"] and j["user"]["email"] == ADMIN["email"]


def test_login_with_invalid_credentials(anon):
    assert anon.req("POST", "/api/auth/login", {"email": ADMIN["email"], "password": "wrong"})[0] == 401
    assert anon.req("POST", "/api/auth/login", {"email": "nobody@example.com", "password": "x"})[0] == 401


def test_login_with_missing_fields(anon):
    assert anon.req("POST", "/api/auth/login", {"email": ADMIN["email"]})[0] in (400, 401, 422)
    assert anon.req("POST", "/api/auth/login", {})[0] in (400, 401, 422)


def test_me_with_valid_missing_and_invalid_token(anon, admin):
    st, j = admin.req("GET", "/api/auth/me")
    assert st == 200 and j["email"] == ADMIN["email"] and j["role"] == "admin" and "password_hash" not in j
    assert anon.req("GET", "/api/auth/me")[0] == 401
    anon.token = "not.a.token"
    assert anon.req("GET", "/api/auth/me")[0] == 401


def test_register_duplicate_email_is_refused(anon):
    assert anon.req("POST", "/api/auth/register", ADMIN)[0] in (403, 409)


def test_refresh_token_gives_a_new_access_token(anon, admin):
    st, j = anon.req("POST", "/api/auth/refresh", {"refresh_token": admin.refresh})
    assert st == 200 and j["access_token"]
    anon.token = j["access_token"]
    assert anon.req("GET", "/api/auth/me")[0] == 200
    assert Client(anon.base.rsplit(":", 1)[1]).req("POST", "/api/auth/refresh", {"refresh_token": "garbage"})[0] == 401


def test_logout(admin):
    assert admin.req("POST", "/api/auth/logout")[0] == 200


def test_mfa_status_and_invalid_totp_code(admin):
    st, j = admin.req("GET", "/api/auth/mfa/recovery/status")
    assert st == 200
    setup = admin.req("POST", "/api/auth/mfa/totp/setup")[1]
    assert setup["secret"] and setup["otpauth_url"].startswith("otpauth://")
    assert admin.req("POST", "/api/auth/mfa/totp/enable", {"code": "000000"})[0] == 400


# ---------------------------------------------------------------------------------------- models
def test_models_require_authentication(anon):
    assert anon.req("GET", "/api/models")[0] == 401 and anon.req("POST", "/api/models", {"name": "x"})[0] == 401


def test_model_create_update_versions_delete(admin):
    assert isinstance(admin.req("GET", "/api/models")[1], list)
    st, m = admin.req("POST", "/api/models", {"name": "unit-model", "description": "first"})
    assert st == 201 and m["name"] == "unit-model"
    st, u = admin.req("PUT", f"/api/models/{m['id']}", {"description": "second"})
    assert st == 200 and u["description"] == "second"
    assert admin.req("GET", f"/api/models/{m['id']}")[1]["description"] == "second"
    assert admin.req("GET", f"/api/models/{m['id']}/versions")[1] == []
    assert admin.req("GET", f"/api/models/{m['id']}/versions/1")[0] == 404
    assert admin.req("DELETE", f"/api/models/{m['id']}")[0] == 200
    assert admin.req("GET", f"/api/models/{m['id']}")[0] == 404


def test_model_not_found(admin):
    assert admin.req("GET", "/api/models/no-such-id")[0] == 404
    assert admin.req("DELETE", "/api/models/no-such-id")[0] == 404
    assert admin.req("PUT", "/api/models/no-such-id", {"description": "x"})[0] == 404


def test_model_needs_a_name(admin):
    assert admin.req("POST", "/api/models", {"description": "nameless"})[0] in (400, 422)


def test_model_tools_inspect_convert_quantize_export(admin):
    import base64

    import torch

    from axonml_b200 import nn
    from axonml_b200.serialize import StateDict
    from axonml_b200.serialize.codec import safetensors_dumps
    net = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 4))
    blob = safetensors_dumps(StateDict.from_module(net).to_tensors())
    m = admin.req("POST", "/api/models", {"name": "tools-model"})[1]
    base = f"/api/models/{m['id']}/versions"
    assert admin.req("POST", base, {"filename": "net.safetensors", "data": base64.b64encode(blob).decode()})[0] == 201
    ins = admin.req("GET", f"{base}/1/inspect")[1]
    assert ins["format"] == "safetensors" and ins["num_parameters"] == 64 * 32 + 32 + 32 * 4 + 4 and ins["num_layers"] == 2
    assert {l["name"]: l["layer_type"] for l in ins["layers"]}["0.weight"] == "Linear" and ins["memory_fp32"].endswith("KB") and ins["trainable_params"] == ins["num_parameters"]
    st, conv = admin.req("POST", f"{base}/1/convert", {"target_format": "json"})
    assert st == 201 and conv["output_format"] == "json" and conv["num_parameters"] == ins["num_parameters"] and conv["version"] == 2
    st, q = admin.req("POST", f"{base}/1/quantize", {"target_type": "Q8_0"})
    assert st == 201 and q["target_type"] == "Q8_0" and q["compression_ratio"] > 2.5 and q["version"] == 3
    assert admin.req("GET", f"{base}/3/inspect")[1]["format"] == "gguf"
    st, ex = admin.req("POST", f"{base}/1/export", {"target": "onnx"})
    assert st == 201 and ex["format"] == "onnx" and "ONNX Runtime" in ex["compatible_with"] and ex["size"] > 0
    from axonml_b200.onnx import import_onnx_bytes
    onnx_model = import_onnx_bytes(admin.req("GET", f"{base}/{ex['version']}/download")[1])
    x = torch.randn(2, 64)
    out = onnx_model.forward({onnx_model.get_inputs()[0].name: x})
    assert torch.allclose(next(iter(out.values())) if isinstance(out, dict) else out, net.eval()(x), atol=1e-5)
    assert admin.req("POST", f"{base}/1/export", {"target": "torchscript"})[0] == 400
    assert admin.req("POST", f"{base}/1/quantize", {"target_type": "Q3_X"})[0] == 400
    assert admin.req("POST", f"{base}/1/convert", {})[0] == 400 and admin.req("GET", f"{base}/99/inspect")[0] == 404
    types = admin.req("GET", "/api/tools/quantization-types")[1]["types"]
    assert {"Q4_0", "Q8_0", "F16"} <= {t["name"] for t in types} and next(t for t in types if t["name"] == "Q4_0")["bits_per_weight"] == 4.5
    admin.req("DELETE", f"/api/models/{m['id']}")


# ------------------------------------------------------------------------------------- inference
def test_inference_endpoints_require_authentication(anon):
    assert anon.req("GET", "/api/inference/endpoints")[0] == 401


def test_inference_endpoint_not_found(admin):
    assert isinstance(admin.req("GET", "/api/inference/endpoints")[1], list)
    assert admin.req("GET", "/api/inference/endpoints/none")[0] == 404
    assert admin.req("DELETE", "/api/inference/endpoints/none")[0] == 404
    assert admin.req("POST", "/api/inference/endpoints/none/start")[0] == 404
    assert admin.req("POST", "/api/inference/predict/none", {"input": [1.0]})[0] == 404


def test_inference_endpoint_needs_an_existing_model(admin):
    assert admin.req("POST", "/api/inference/endpoints", {"name": "ep", "model_id": "missing", "version": 1})[0] in (400, 404)


def test_inference_overview(admin):
    st, j = admin.req("GET", "/api/status/inference")
    assert st == 200 and "endpoints_running" in j


# -------------------------------------------------------------------------------------- training
def test_training_runs_require_authentication(anon):
    assert anon.req("GET", "/api/training/runs")[0] == 401


def test_training_run_not_found(admin):
    assert admin.req("GET", "/api/training/runs/none")[0] == 404
    assert admin.req("DELETE", "/api/training/runs/none")[0] == 404
    assert admin.req("GET", "/api/training/runs/none/metrics")[0] == 404


def test_training_run_lifecycle_with_posted_metrics_and_logs(admin):
    st, run = admin.req("POST", "/api/training/runs", {"name": "unit-run", "model_type": "mlp", "config": {"epochs": 1}, "start": False})
    assert st == 201 and run["name"] == "unit-run" and run["status"] == "pending"        # start=False: tracked for an outside trainer
    rid = run["id"]
    for step in range(3):
        assert admin.req("POST", f"/api/training/runs/{rid}/metrics", {"epoch": 0, "step": step, "loss": 1.0 / (step + 1)})[0] in (200, 201)
    assert admin.req("POST", f"/api/training/runs/{rid}/logs", {"level": "info", "message": "hello from the test"})[0] in (200, 201)
    metrics = admin.req("GET", f"/api/training/runs/{rid}/metrics")[1]
    assert len(metrics) == 3 and metrics[-1]["loss"] == pytest.approx(1 / 3)
    logs = admin.req("GET", f"/api/training/runs/{rid}/logs")[1]
    assert any("hello from the test" in l["message"] for l in logs)
    assert admin.req("POST", f"/api/training/runs/{rid}/complete", {})[0] == 200
    assert admin.req("GET", f"/api/training/runs/{rid}")[1]["status"] == "completed"
    assert admin.req("DELETE", f"/api/training/runs/{rid}")[0] == 200


def test_training_run_stop_pagination_and_filtering(admin):
    ids = []
    for i in range(3):
        st, run = admin.req("POST", "/api/training/runs", {"name": f"page-{i}", "model_type": "mlp", "start": False})
        assert st == 201
        ids.append(run["id"])
    assert admin.req("POST", f"/api/training/runs/{ids[0]}/stop")[1] == {"stopping": True}
    for _ in range(100):                                   # the trainer thread notices the request between batches
        if admin.req("GET", f"/api/training/runs/{ids[0]}")[1]["status"] == "stopped":
            break
        time.sleep(0.1)
    page = admin.req("GET", "/api/training/runs?limit=2")[1]
    assert len(page) == 2
    rest = admin.req("GET", "/api/training/runs?limit=2&offset=2")[1]
    assert {r["id"] for r in page}.isdisjoint({r["id"] for r in rest})
    stopped = admin.req("GET", "/api/training/runs?status=stopped")[1]
    assert all(r["status"] == "stopped" for r in stopped) and ids[0] in {r["id"] for r in stopped}
    for i in ids:
        admin.req("DELETE", f"/api/training/runs/{i}")


# ----------------------------------------------------------------------------------------- admin
def test_admin_routes_need_the_admin_role(anon, admin):
    assert anon.req("GET", "/api/admin/users")[0] == 401
    st, u = admin.req("POST", "/api/admin/users", {"email": "user@example.com", "name": "User", "password": "user-pass-123", "role": "user"})
    assert st == 201 and u["role"] == "user"
    c = Client(anon.base.rsplit(":", 1)[1])
    c.token = c.req("POST", "/api/auth/login", {"email": "user@example.com", "password": "user-pass-123"})[1]["access_token"]
    assert c.req("GET", "/api/admin/users")[0] == 403 and c.req("GET", "/api/models")[0] == 200
    assert admin.req("DELETE", f"/api/admin/users/{u['id']}")[0] == 200


def test_admin_user_management(admin):
    users = admin.req("GET", "/api/admin/users")[1]
    me = next(u for u in users if u["email"] == ADMIN["email"])
    assert admin.req("GET", f"/api/admin/users/{me['id']}")[1]["email"] == ADMIN["email"]
    assert admin.req("GET", "/api/admin/users/none")[0] == 404
    st, u = admin.req("POST", "/api/admin/users", {"email": "viewer@example.com", "name": "V", "password": "viewer-pass-1", "role": "viewer"})
    assert st == 201
    assert admin.req("POST", "/api/admin/users", {"email": "viewer@example.com", "name": "V", "password": "viewer-pass-1"})[0] == 409
    assert admin.req("PUT", f"/api/admin/users/{u['id']}", {"role": "user"})[1]["role"] == "user"
    assert admin.req("DELETE", f"/api/admin/users/{me['id']}")[0] in (400, 403, 409)          # not oneself
    assert admin.req("DELETE", f"/api/admin/users/{u['id']}")[0] == 200
    assert admin.req("GET", "/api/admin/stats")[0] == 200


def test_admin_query_reads_a_collection(admin):
    admin.req("POST", "/api/models", {"name": "queried-model"})
    st, j = admin.req("POST", "/api/admin/query", {"collection": "models", "filter": {"name": "queried-model"}})
    assert st == 200 and [d["name"] for d in j["rows"]] == ["queried-model"] and j["affected_rows"] == 1
    assert admin.req("POST", "/api/admin/query", {"collection": "users"})[0] == 403       # password hashes stay inside
    assert admin.req("POST", "/api/admin/query", {"collection": "no_such_collection"})[0] in (400, 404)


# ---------------------------------------------------------------------------------------- system
def test_system_routes(anon, admin):
    assert anon.req("GET", "/api/system/info")[0] == 401
    info = admin.req("GET", "/api/system/info")[1]
    assert info["cpu_count"] >= 1 and info["total_memory_bytes"] > 0 and info["framework"] == "axonml_b200"
    assert admin.req("GET", "/api/system/metrics")[0] == 200 and isinstance(admin.req("GET", "/api/system/gpus")[1], list)
    assert admin.req("GET", "/api/system/metrics/history")[0] == 200
    assert admin.req("GET", "/api/status/pool")[0] == 200 and admin.req("GET", "/api/status/cache")[0] == 200
    assert b"axonml_" in anon.req("GET", "/metrics")[1]


# -------------------------------------------------------------------------------------- datasets
def test_dataset_routes_require_authentication(anon):
    for method, path in (("GET", "/api/datasets"), ("POST", "/api/data/x/analyze"), ("POST", "/api/data/x/preview"),
                         ("POST", "/api/data/x/validate"), ("POST", "/api/data/x/generate-config"), ("GET", "/api/builtin-datasets"),
                         ("GET", "/api/kaggle/status"), ("GET", "/api/kaggle/search?query=mnist")):
        assert anon.req(method, path, {} if method == "POST" else None)[0] == 401, path


def test_dataset_not_found_and_builtin_catalogue(admin):
    assert admin.req("POST", "/api/data/none/analyze", {})[0] == 404 and admin.req("GET", "/api/datasets/none")[0] == 404
    builtin = admin.req("GET", "/api/builtin-datasets")[1]
    assert {"mnist", "cifar-10", "iris"} <= {d["id"] for d in builtin}
    found = admin.req("GET", "/api/builtin-datasets/search?query=cifar")[1]
    assert [d["id"] for d in found] == ["cifar-10", "cifar-100"]
    assert {s["id"] for s in admin.req("GET", "/api/builtin-datasets/sources")[1]} >= {"builtin", "kaggle", "uci"}
    assert admin.req("GET", "/api/builtin-datasets/mnist")[1]["classes"] == 10
    assert admin.req("GET", "/api/builtin-datasets/nonexistent-id")[0] == 404
    assert admin.req("POST", "/api/builtin-datasets/nonexistent-id/prepare", {})[0] == 404
    assert "loading_code" in admin.req("POST", "/api/builtin-datasets/iris/prepare", {})[1]


def test_kaggle_status_and_search_without_credentials(admin):
    st, j = admin.req("GET", "/api/kaggle/status")
    assert st == 200 and j["configured"] is False
    assert admin.req("GET", "/api/kaggle/search?query=mnist")[0] == 403
    assert admin.req("GET", "/api/kaggle/downloaded")[1] == []
    assert admin.req("POST", "/api/kaggle/credentials", {"username": ""})[0] in (400, 422)


# ------------------------------------------------------------------------------------------- hub
def test_hub_browse(admin):
    models = admin.req("GET", "/api/hub/models")[1]
    assert any(m["name"] == "resnet18" for m in models)
    info = admin.req("GET", "/api/hub/models/resnet18")[1]
    assert info["architecture"] == "ResNet" and info["parameters"] > 11_000_000 and info["cached"] is False
    assert admin.req("GET", "/api/hub/models/no-such-model")[0] == 404
    assert admin.req("GET", "/api/hub/cache")[0] == 200


# ---------------------------------------------------------------------------------------- errors
def test_invalid_json_missing_route_and_wrong_method(admin):
    assert admin.req("POST", "/api/models", raw=b"{not json", ctype="application/json")[0] == 400
    assert admin.req("GET", "/api/no/such/route")[0] == 404
    assert admin.req("DELETE", "/health")[0] in (404, 405)


def test_concurrent_requests_are_all_answered(srv, admin):
    def one(_):
        r = urllib.request.Request(f"http://127.0.0.1:{srv.port}/api/models", headers={"Authorization": "Bearer " + admin.token})
        with urllib.request.urlopen(r, timeout=30) as resp:
            return resp.status, json.loads(resp.read())
    with cf.ThreadPoolExecutor(8) as pool:
        out = list(pool.map(one, range(24)))
    assert all(st == 200 and isinstance(body, list) for st, body in out)
