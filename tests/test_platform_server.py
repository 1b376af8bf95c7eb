"""Platform server: document store, authentication primitives and the REST/WebSocket API end to
end over a real socket (CPU only)."""
import base64
import json
import os
import time
import urllib.error
import urllib.request

import pytest
import torch

from axonml_b200.server.app import (DocumentStore, JwtAuth, NotFound, PlatformServer, RecoveryAuth, TotpAuth, hash_password,
                                    verify_password)
from axonml_b200.server.app import websocket as WS
from axonml_b200.server.app.auth import AuthError


# ----------------------------------------------------------------------------- store
def test_document_store_persists_and_filters(tmp_path):
    s = DocumentStore(str(tmp_path))
    runs = s["runs"]
    a = runs.insert({"name": "a", "step": 1, "meta": {"k": 3}})
    runs.insert({"name": "b", "step": 5})
    runs.insert({"name": "c", "step": 9})
    assert runs.count() == 3
    assert [d["name"] for d in runs.find({"step": {"$gte": 5}}, sort="step")] == ["b", "c"]
    assert runs.find_one(name="a")["id"] == a["id"]
    assert runs.find({"meta.k": 3})[0]["name"] == "a"
    runs.update(a["id"], {"step": 2})
    s.kv_set("answer", 42)
    s2 = DocumentStore(str(tmp_path))                  # a restart sees the same data
    assert s2["runs"].get(a["id"])["step"] == 2 and s2.kv_get("answer") == 42
    s2["runs"].delete(a["id"])
    with pytest.raises(NotFound):
        s2["runs"].get(a["id"])
    assert s2["runs"].delete_where({"step": {"$gt": 0}}) == 2


# ----------------------------------------------------------------------------- auth primitives
def test_password_hash_and_jwt_roundtrip():
    h = hash_password("correct horse")
    assert verify_password("correct horse", h) and not verify_password("wrong", h)
    jwt = JwtAuth("0123456789abcdef0123", access_expiry_hours=1)
    pair = jwt.create_token_pair("u1", "a@b.c", "admin")
    c = jwt.validate_access_token(pair["access_token"])
    assert (c.sub, c.email, c.role, c.token_type) == ("u1", "a@b.c", "admin", "access")
    with pytest.raises(AuthError):
        jwt.validate_access_token(pair["refresh_token"])           # wrong token type
    with pytest.raises(AuthError):
        jwt.validate_access_token(pair["access_token"][:-3] + "abc")  # bad signature
    with pytest.raises(AuthError):
        JwtAuth("another-secret-0123456789").validate_access_token(pair["access_token"])
    expired = JwtAuth("0123456789abcdef0123", access_expiry_hours=-1).create_access_token("u", "e", "user")
    with pytest.raises(AuthError, match="expired"):
        jwt.validate_access_token(expired)
    assert jwt.validate_access_token(jwt.refresh_access_token(pair["refresh_token"])["access_token"]).sub == "u1"
    assert JwtAuth.extract_from_header("Bearer abc") == "abc" and JwtAuth.extract_from_header("Basic x") is None


def test_totp_matches_rfc6238_vectors():
    # RFC 6238 appendix B, SHA-1, secret "12345678901234567890", 8 digits
    secret = base64.b32encode(b"12345678901234567890").decode()
    t8 = TotpAuth(digits=8)
    assert t8.code_at(secret, 59) == "94287082"
    assert t8.code_at(secret, 1111111109) == "07081804"
    assert t8.code_at(secret, 1234567890) == "89005924"
    t = TotpAuth()
    s = t.setup("user@example.com")
    assert s["otpauth_url"].startswith("otpauth://totp/AxonML:user%40example.com?secret=" + s["secret"])
    now = 1_700_000_000
    assert t.verify(s["secret"], t.code_at(s["secret"], now), now)
    assert t.verify(s["secret"], t.code_at(s["secret"], now - 30), now)          # one step of drift
    assert not t.verify(s["secret"], t.code_at(s["secret"], now - 90), now)


def test_recovery_codes_are_single_use_hashes():
    rc = RecoveryAuth.generate_codes(4)
    assert len(rc["codes"]) == 4 and all(len(c) == 11 and c[5] == "-" for c in rc["codes"])
    assert all(c not in h for c, h in zip(rc["codes"], rc["hashed_codes"]))
    assert RecoveryAuth.verify_code(rc["codes"][2], rc["hashed_codes"]) == 2
    assert RecoveryAuth.verify_code(rc["codes"][2].replace("-", ""), rc["hashed_codes"]) == 2
    assert RecoveryAuth.verify_code("00000-00000", rc["hashed_codes"]) in (None, 0, 1, 2, 3)
    assert RecoveryAuth.verify_code("nonsense", rc["hashed_codes"]) is None


# ----------------------------------------------------------------------------- HTTP end to end
class Client:
    def __init__(self, port):
        self.base, self.token = f"http://127.0.0.1:{port}", None

    def req(self, method, path, body=None, raw=None, ctype="application/json"):
        data = raw if raw is not None else (json.dumps(body).encode() if body is not None else None)
        r = urllib.request.Request(self.base + path, data=data, method=method)
        if data is not None:
            r.add_header("Content-Type", ctype)
        if self.token:
            r.add_header("Authorization", "Bearer " + self.token)
        try:
            with urllib.request.urlopen(r, timeout=30) as resp:
                payload, status, ct = resp.read(), resp.status, resp.headers.get("Content-Type", "")
        except urllib.error.HTTPError as e:
            payload, status, ct = e.read(), e.code, e.headers.get("Content-Type", "")
        return status, (json.loads(payload) if ct.startswith("application/json") else payload)


@pytest.fixture()
def server(tmp_path):
    s = PlatformServer(port=0, data_dir=str(tmp_path / "srv")).start()
    yield s
    s.stop()


def _login(c, email="ada@example.com", password="s3cret-pass"):
    st, j = c.req("POST", "/api/auth/login", {"email": email, "password": password})
    assert st == 200, j
    return j


def test_auth_flow_with_totp_and_recovery(server):
    c = Client(server.port)
    assert c.req("GET", "/health")[1]["status"] == "healthy"
    assert c.req("GET", "/api/auth/me")[0] == 401
    st, j = c.req("POST", "/api/auth/register", {"email": "Ada@example.com", "name": "Ada", "password": "s3cret-pass"})
    assert st == 201 and j["user"]["role"] == "admin"             # first account administers
    # by default only the first account may register itself; later accounts come from the administrator
    assert c.req("POST", "/api/auth/register", {"email": "bob@example.com", "name": "x", "password": "s3cret-pass"})[0] == 403
    assert c.req("POST", "/api/auth/login", {"email": "ada@example.com", "password": "nope"})[0] == 401
    j = _login(c)
    c.token = j["access_token"]
    assert c.req("GET", "/api/auth/me")[1]["email"] == "ada@example.com"
    # second factor
    setup = c.req("POST", "/api/auth/mfa/totp/setup")[1]
    assert c.req("POST", "/api/auth/mfa/totp/enable", {"code": "000000"})[0] in (400, 200)
    en = c.req("POST", "/api/auth/mfa/totp/enable", {"code": TotpAuth().code_at(setup["secret"])})[1]
    assert en["mfa_enabled"] and len(en["recovery_codes"]) == 10
    c.token = None
    j = _login(c)
    assert j["requires_mfa"] and "access_token" not in j
    assert c.req("POST", "/api/auth/mfa/totp/verify", {"mfa_token": j["mfa_token"], "code": "123"})[0] == 401
    ok = c.req("POST", "/api/auth/mfa/totp/verify", {"mfa_token": j["mfa_token"], "code": TotpAuth().code_at(setup["secret"])})
    assert ok[0] == 200 and ok[1]["access_token"]
    j = _login(c)
    rec = c.req("POST", "/api/auth/mfa/recovery", {"mfa_token": j["mfa_token"], "code": en["recovery_codes"][0]})
    assert rec[0] == 200 and rec[1]["recovery_codes_left"] == 9
    j = _login(c)
    assert c.req("POST", "/api/auth/mfa/recovery", {"mfa_token": j["mfa_token"], "code": en["recovery_codes"][0]})[0] == 401
    # refresh, logout revokes
    c.token = rec[1]["access_token"]
    new = c.req("POST", "/api/auth/refresh", {"refresh_token": rec[1]["refresh_token"]})[1]
    assert new["access_token"]
    assert c.req("POST", "/api/auth/logout")[0] == 200
    assert c.req("GET", "/api/auth/me")[0] == 401
    c.token = new["access_token"]
    assert c.req("POST", "/api/auth/mfa/disable", {"password": "s3cret-pass"})[1] == {"mfa_enabled": False}
    # administration and roles
    st, u2 = c.req("POST", "/api/admin/users", {"email": "bob@example.com", "name": "Bob", "password": "bobs-password"})
    assert st == 201 and u2["role"] == "user"
    assert len(c.req("GET", "/api/admin/users")[1]) == 2
    assert c.req("GET", "/api/admin/stats")[1]["users"] == 2
    bob = Client(server.port)
    bob.token = _login(bob, "bob@example.com", "bobs-password")["access_token"]
    assert bob.req("GET", "/api/admin/users")[0] == 403
    assert c.req("POST", "/api/admin/query", {"collection": "users"})[0] == 403
    assert c.req("DELETE", f"/api/admin/users/{u2['id']}")[1] == {"deleted": True}
    assert c.req("GET", "/nope")[0] == 404 and c.req("DELETE", "/health")[0] == 405


def _admin(server):
    c = Client(server.port)
    c.req("POST", "/api/auth/register", {"email": "ada@example.com", "name": "Ada", "password": "s3cret-pass"})
    c.token = _login(c)["access_token"]
    return c


def test_training_run_streams_metrics_over_websocket(server):
    c = _admin(server)
    st, run = c.req("POST", "/api/training/runs", {"name": "mnist-mlp", "model_type": "mlp", "start": False,
                                                   "config": {"epochs": 1, "steps_per_epoch": 16, "log_every": 4, "device": "cpu"}})
    assert st == 201 and run["status"] == "pending" and run["config"]["optimizer"] == "adam"
    ws = WS.connect("127.0.0.1", server.port, f"/api/training/runs/{run['id']}/stream?token={c.token}")
    assert json.loads(ws.recv(5))["data"]["status"] == "pending"
    server.executor.start(server.runs.get(run["id"]))
    kinds, losses = [], []
    t0 = time.time()
    while time.time() - t0 < 90:
        m = ws.recv(1.0)
        if m is None:
            continue
        m = json.loads(m)
        kinds.append(m["type"])
        if m["type"] == "metrics":
            losses.append(m["data"]["loss"])
        elif m["data"]["status"] in ("completed", "failed"):
            final = m["data"]["status"]
            break
    ws.close()
    assert final == "completed", c.req("GET", f"/api/training/runs/{run['id']}/logs")[1]
    assert len(losses) == 4 and all(torch.isfinite(torch.tensor(losses)))
    got = c.req("GET", f"/api/training/runs/{run['id']}")[1]
    assert got["status"] == "completed" and got["latest_metrics"]["step"] == 16 and os.path.exists(got["artifact"])
    hist = c.req("GET", f"/api/training/runs/{run['id']}/metrics?start_step=8")[1]
    assert [m["step"] for m in hist] == [8, 12, 16]
    assert any("epoch 1 done" in l["message"] for l in c.req("GET", f"/api/training/runs/{run['id']}/logs")[1])
    # an external trainer reports into a run it created
    st, ext = c.req("POST", "/api/training/runs", {"name": "external", "model_type": "custom", "start": False})
    assert c.req("POST", f"/api/training/runs/{ext['id']}/metrics", {"epoch": 1, "step": 3, "loss": 0.5})[0] == 200
    assert c.req("GET", f"/api/training/runs/{ext['id']}")[1]["status"] == "running"
    assert c.req("POST", f"/api/training/runs/{ext['id']}/stop")[0] == 200
    assert c.req("GET", f"/api/training/runs/{ext['id']}")[1]["status"] == "stopped"
    assert c.req("DELETE", f"/api/training/runs/{ext['id']}")[1] == {"deleted": True}
    assert len(c.req("GET", "/api/training/runs")[1]) == 1


def test_models_datasets_endpoints_and_prediction(server, tmp_path):
    from axonml_b200 import nn
    from axonml_b200.serialize import save_state_dict
    from axonml_b200.serialize.state_dict import StateDict
    c = _admin(server)
    st, m = c.req("POST", "/api/models", {"name": "tiny", "description": "2-layer MLP"})
    assert st == 201 and c.req("POST", "/api/models", {"name": "tiny"})[0] == 409
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 3))
    path = str(tmp_path / "tiny.axonml")
    save_state_dict(StateDict.from_module(net), path)
    blob = open(path, "rb").read()
    st, v = c.req("POST", f"/api/models/{m['id']}/versions?filename=tiny.axonml", raw=blob, ctype="application/octet-stream")
    assert st == 201 and v["version"] == 1 and v["format"] == "axonml" and v["file_size"] == len(blob)
    st, v2 = c.req("POST", f"/api/models/{m['id']}/versions", {"filename": "tiny.axonml", "data": base64.b64encode(blob).decode()})
    assert v2["version"] == 2 and c.req("GET", f"/api/models/{m['id']}")[1]["latest_version"] == 2
    assert c.req("GET", f"/api/models/{m['id']}/versions/1/download")[1] == blob
    assert c.req("POST", f"/api/models/{m['id']}/versions/2/deploy")[1]["deployed"] is True
    assert c.req("GET", "/api/public/models")[1][0]["name"] == "tiny"
    # endpoint lifecycle + prediction against the torch module
    st, ep = c.req("POST", "/api/inference/endpoints", {"name": "tiny-ep", "model_id": m["id"], "version": 1})
    assert st == 201 and ep["status"] == "stopped"
    assert c.req("POST", "/api/inference/predict/tiny-ep", {"input": [1, 2, 3, 4]})[0] == 404
    assert c.req("POST", f"/api/inference/endpoints/{ep['id']}/start")[1]["status"] == "running"
    out = c.req("POST", "/api/inference/predict/tiny-ep", {"input": [1.0, 2.0, 3.0, 4.0]})[1]
    want = net(torch.tensor([[1.0, 2.0, 3.0, 4.0]])).detach()[0]
    assert torch.allclose(torch.tensor(out["output"]), want, atol=1e-4)
    assert c.req("GET", f"/api/inference/endpoints/{ep['id']}/info")[1]["parameters"] == 4 * 8 + 8 + 8 * 3 + 3
    assert c.req("GET", f"/api/inference/endpoints/{ep['id']}/metrics")[1]["success"] >= 1
    assert b"axonml_" in c.req("GET", "/api/metrics")[1]
    assert c.req("POST", f"/api/inference/endpoints/{ep['id']}/stop")[1]["status"] == "stopped"
    assert c.req("GET", "/api/status/inference")[1]["endpoints_running"] == 0
    # datasets: upload, analyse, preview, validate, config
    csv = "a,b,label\n" + "\n".join(f"{i},{i * 0.5},{'x' if i % 4 else 'y'}" for i in range(40)) + "\n1,,x\n"
    st, ds = c.req("POST", "/api/datasets?filename=toy.csv&name=toy", raw=csv.encode(), ctype="text/csv")
    assert st == 201 and ds["num_samples"] == 41 and ds["num_features"] == 3
    an = c.req("POST", f"/api/data/{ds['id']}/analyze", {})[1]
    assert an["dataset_type"] == "tabular" and an["num_classes"] == 2 and an["missing_values"] == 1
    assert an["class_counts"] == {"x": 31, "y": 10} and an["recommendations"]["architecture"] == "mlp"
    assert len(c.req("POST", f"/api/data/{ds['id']}/preview", {"num_samples": 3})[1]["samples"]) == 3
    val = c.req("POST", f"/api/data/{ds['id']}/validate", {"num_classes": 3})[1]
    assert not val["valid"] and "expected 3 classes" in val["issues"][0] and any("imbalance" in w for w in val["warnings"])
    cfg = c.req("POST", f"/api/data/{ds['id']}/generate-config", {})[1]["config"]
    import tomllib
    assert tomllib.loads(cfg)["model"]["architecture"] == "mlp"
    assert c.req("DELETE", f"/api/datasets/{ds['id']}")[1] == {"deleted": True}
    assert c.req("DELETE", f"/api/models/{m['id']}")[1] == {"deleted": True}
    assert [d["id"] for d in c.req("GET", "/api/builtin-datasets")[1]][:2] == ["mnist", "fashion-mnist"]


def test_notebooks_execute_python_cells_and_roundtrip_ipynb(server):
    c = _admin(server)
    st, nb = c.req("POST", "/api/notebooks", {"name": "scratch"})
    assert st == 201 and [x["cell_type"] for x in nb["cells"]] == ["markdown", "code"]
    code = nb["cells"][1]["id"]
    c.req("PUT", f"/api/notebooks/{nb['id']}/cells/{code}", {"source": "x = 6 * 7\nprint('hello')\nx"})
    cell = c.req("POST", f"/api/notebooks/{nb['id']}/cells/{code}/execute")[1]
    assert cell["status"] == "completed" and cell["outputs"][0]["text"] == "hello\n" and cell["outputs"][1]["text"] == "42"
    st, c2 = c.req("POST", f"/api/notebooks/{nb['id']}/cells", {"cell_type": "code", "source": "x + 1"})
    assert c.req("POST", f"/api/notebooks/{nb['id']}/cells/{c2['id']}/execute")[1]["outputs"][0]["text"] == "43"   # shared namespace
    st, c3 = c.req("POST", f"/api/notebooks/{nb['id']}/cells", {"source": "1 / 0"})
    bad = c.req("POST", f"/api/notebooks/{nb['id']}/cells/{c3['id']}/execute")[1]
    assert bad["status"] == "error" and bad["outputs"][-1]["error_name"] == "ZeroDivisionError"
    ck = c.req("POST", f"/api/notebooks/{nb['id']}/checkpoints", {"label": "before delete"})[1]
    c.req("DELETE", f"/api/notebooks/{nb['id']}/cells/{c3['id']}")
    assert len(c.req("GET", f"/api/notebooks/{nb['id']}")[1]["cells"]) == 3
    assert len(c.req("POST", f"/api/notebooks/{nb['id']}/checkpoints/{ck['id']}/restore")[1]["cells"]) == 4
    ipynb = c.req("GET", f"/api/notebooks/{nb['id']}/export")[1]
    assert ipynb["nbformat"] == 4 and ipynb["cells"][1]["outputs"][0]["output_type"] == "stream"
    st, imp = c.req("POST", "/api/notebooks/import", {"notebook": ipynb, "name": "copy"})
    assert st == 201 and [x["source"] for x in imp["cells"]] == [x["source"] for x in c.req("GET", f"/api/notebooks/{nb['id']}")[1]["cells"]]
    assert c.req("POST", f"/api/notebooks/{nb['id']}/ai-assist", {"prompt": "hi"})[0] == 503
    assert c.req("DELETE", f"/api/notebooks/{nb['id']}")[1] == {"deleted": True}


def test_system_hub_kaggle_terminal_and_dashboard(server):
    c = _admin(server)
    info = c.req("GET", "/api/system/info")[1]
    assert info["cpu_count"] >= 1 and info["framework"] == "axonml_b200" and isinstance(info["gpus"], list)
    m = c.req("GET", "/api/system/metrics")[1]
    assert 0.0 <= m["cpu_percent"] <= 100.0
    assert len(c.req("GET", "/api/system/metrics/history")[1]) >= 1
    b = c.req("POST", "/api/system/benchmark", {"size": 64, "iterations": 2, "device": "cpu"})[1]
    assert b["matmul_gflops"] > 0 and b["copy_gb_per_s"] > 0
    hub = c.req("GET", "/api/hub/models")[1]
    assert any(h["name"] == "lenet" for h in hub) or len(hub) > 3
    assert c.req("GET", "/api/hub/models/not-a-model")[0] == 404
    assert c.req("GET", "/api/kaggle/status")[1]["configured"] is False
    assert c.req("POST", "/api/kaggle/credentials", {"username": "u", "key": "k"})[1] == {"configured": True}
    assert c.req("GET", "/api/kaggle/status")[1]["username"] == "u"
    assert c.req("GET", "/api/kaggle/search?q=mnist")[0] in (200, 503)          # 503 without a route to kaggle.com
    assert c.req("GET", "/api/terminal/info")[1]["enabled"] is False
    assert c.req("GET", "/api/terminal")[0] == 403
    page = c.req("GET", "/")[1]
    assert b"<title>AxonML</title>" in page and b"/api/training/runs" in page


def test_open_registration_rejects_a_duplicate_address(tmp_path):
    s = PlatformServer(port=0, data_dir=str(tmp_path / "srv"), allow_registration=True).start()
    try:
        c = Client(s.port)
        assert c.req("POST", "/api/auth/register", {"email": "Ada@example.com", "name": "Ada", "password": "s3cret-pass"})[0] == 201
        assert c.req("POST", "/api/auth/register", {"email": "ada@example.com", "name": "x", "password": "s3cret-pass"})[0] == 409
        st, j = c.req("POST", "/api/auth/register", {"email": "bob@example.com", "name": "Bob", "password": "s3cret-pass"})
        assert st == 201 and j["user"]["role"] == "user"
    finally:
        s.stop()


def test_notebook_cells_run_outside_the_server_process(server):
    """A cell sees neither the server's process nor its environment, output of one notebook never
    lands in another, a viewer may not run code, and a cell that does not end is cut off."""
    import os
    from axonml_b200.server.app.notebooks import NotebookKernel
    c = Client(server.port)
    c.req("POST", "/api/auth/register", {"email": "ada@example.com", "name": "Ada", "password": "s3cret-pass"})
    c.token = _login(c)["access_token"]
    nb = c.req("POST", "/api/notebooks", {"name": "iso"})[1]
    code = nb["cells"][1]["id"]
    c.req("PUT", f"/api/notebooks/{nb['id']}/cells/{code}", {"source": "import os\nos.getpid()"})
    cell = c.req("POST", f"/api/notebooks/{nb['id']}/cells/{code}/execute")[1]
    assert cell["status"] == "completed" and int(cell["outputs"][0]["text"]) != os.getpid()
    os.environ["AXONML_TEST_SECRET"] = "hunter2"
    try:
        k = NotebookKernel(timeout_s=20)
        out, ok = k.execute("import os\nos.environ.get('AXONML_TEST_SECRET')")
        assert ok and out == []                                        # None: the variable is not passed on
        out, ok = k.execute("print('a'); 1 + 1")
        assert ok and out[0]["text"] == "a\n" and out[1]["text"] == "2"
        k.close()
    finally:
        del os.environ["AXONML_TEST_SECRET"]
    slow = NotebookKernel(timeout_s=1.0)
    out, ok = slow.execute("import time\ntime.sleep(30)")
    assert not ok and out[0]["error_name"] == "CellTimeout"
    out, ok = slow.execute("41 + 1")                                   # a fresh kernel process answers
    assert ok and out[0]["text"] == "42"
    slow.close()
    # a viewer owns a notebook but may not run code
    admin = c
    st, v = admin.req("POST", "/api/admin/users", {"email": "vi@example.com", "name": "Vi", "password": "s3cret-pass", "role": "viewer"})
    assert st in (200, 201), v
    cv = Client(server.port)
    cv.token = _login(cv, "vi@example.com")["access_token"]
    nbv = cv.req("POST", "/api/notebooks", {"name": "mine"})[1]
    assert cv.req("POST", f"/api/notebooks/{nbv['id']}/cells/{nbv['cells'][1]['id']}/execute")[0] == 403
    assert cv.req("POST", f"/api/notebooks/{nbv['id']}/run-all")[0] == 403


# ----------------------------------------------------------------------------- WebAuthn
def test_webauthn_primitives_reject_tampering():
    from axonml_b200.server.app import webauthn as W
    assert W.cbor_decode(W.cbor_encode({"a": [1, -5, b"xy", "t", None, True, 70000], -2: {1: 2}}))[0] == \
        {"a": [1, -5, b"xy", "t", None, True, 70000], -2: {1: 2}}
    rp = W.WebAuthnAuth("localhost", "AxonML", "http://localhost:3021")
    key = W.SoftwareAuthenticator("http://localhost:3021")
    cred = rp.finish_registration("u1", key.create(rp.start_registration("u1", "a@b.c", "Ada")), "yubikey")
    assert cred["name"] == "yubikey" and cred["counter"] == 0 and len(W.b64u_dec(cred["public_key"])) == 64
    # a good assertion, then the same one replayed (challenge is single use)
    resp = key.get(rp.start_authentication("u1", [cred]))
    cred2 = rp.finish_authentication("u1", resp, [cred])
    assert cred2["counter"] == 1
    with pytest.raises(W.WebAuthnError, match="pending"):
        rp.finish_authentication("u1", resp, [cred2])
    # tampered signature, wrong origin, stale counter, unknown credential
    resp = key.get(rp.start_authentication("u1", [cred2]))
    bad = json.loads(json.dumps(resp))
    sig = bytearray(W.b64u_dec(bad["response"]["signature"]))
    sig[-1] ^= 1
    bad["response"]["signature"] = W.b64u(bytes(sig))
    with pytest.raises(W.WebAuthnError, match="signature"):
        rp.finish_authentication("u1", bad, [cred2])
    evil = W.SoftwareAuthenticator("http://evil.example")
    evil._keys, evil._counter = key._keys, 10
    with pytest.raises(W.WebAuthnError, match="origin"):
        rp.finish_authentication("u1", evil.get(rp.start_authentication("u1", [cred2])), [cred2])
    with pytest.raises(W.WebAuthnError, match="counter"):
        rp.finish_authentication("u1", key.get(rp.start_authentication("u1", [cred2])), [{**cred2, "counter": 99}])
    other = W.SoftwareAuthenticator("http://localhost:3021")
    other_cred = rp.finish_registration("u2", other.create(rp.start_registration("u2", "x@y.z", "X")), "")
    with pytest.raises(W.WebAuthnError, match="unknown credential"):
        rp.finish_authentication("u1", other.get(rp.start_authentication("u1", [other_cred])), [cred2])
    # registration with a client-data type of the other ceremony
    opts = rp.start_registration("u3", "q@r.s", "Q")
    wrong = key.create(opts)
    cd = json.loads(W.b64u_dec(wrong["response"]["client_data_json"]))
    cd["type"] = "webauthn.get"
    wrong["response"]["client_data_json"] = W.b64u(json.dumps(cd).encode())
    with pytest.raises(W.WebAuthnError, match="type"):
        rp.finish_registration("u3", wrong, "")


def test_webauthn_second_factor_over_http(server):
    from axonml_b200.server.app import webauthn as W
    c = Client(server.port)
    c.req("POST", "/api/auth/register", {"email": "ada@example.com", "name": "Ada", "password": "s3cret-pass"})
    c.token = _login(c)["access_token"]
    key = W.SoftwareAuthenticator(server.public_url)
    st, opts = c.req("POST", "/api/auth/mfa/webauthn/register/start")
    assert st == 200 and opts["rp"]["id"] == "localhost" and opts["pub_key_cred_params"][0]["alg"] == -7
    st, out = c.req("POST", "/api/auth/mfa/webauthn/register/finish", {"credential": key.create(opts), "name": "laptop key"})
    assert st == 201 and out["webauthn_enabled"]
    assert c.req("GET", "/api/auth/me")[1]["webauthn_enabled"] is True
    assert [k["name"] for k in c.req("GET", "/api/auth/mfa/webauthn/credentials")[1]] == ["laptop key"]
    c.token = None
    j = _login(c)
    assert j["requires_mfa"] and j["mfa_methods"] == ["webauthn"]
    st, ch = c.req("POST", "/api/auth/mfa/webauthn/authenticate/start", {"mfa_token": j["mfa_token"]})
    assert st == 200 and ch["allow_credentials"][0]["id"] == out["credential"]["credential_id"]
    assertion = key.get(ch)
    forged = json.loads(json.dumps(assertion))
    forged["response"]["authenticator_data"] = W.b64u(W.b64u_dec(forged["response"]["authenticator_data"])[:-1] + b"\x09")
    assert c.req("POST", "/api/auth/mfa/webauthn/authenticate/finish", {"mfa_token": j["mfa_token"], "credential": forged})[0] == 400
    st, ch = c.req("POST", "/api/auth/mfa/webauthn/authenticate/start", {"mfa_token": j["mfa_token"]})
    st, ok = c.req("POST", "/api/auth/mfa/webauthn/authenticate/finish", {"mfa_token": j["mfa_token"], "credential": key.get(ch)})
    assert st == 200 and ok["access_token"]
    c.token = ok["access_token"]
    cid = out["credential"]["credential_id"]
    assert c.req("DELETE", f"/api/auth/mfa/webauthn/credentials/{cid}")[1] == {"deleted": True, "webauthn_enabled": False}


# ----------------------------------------------------------------------------- external services (faked over HTTP)
class _Fake:
    """A tiny HTTP server that records requests and answers from a table of (method, path prefix)."""

    def __init__(self, routes):
        import http.server
        import threading
        fake = self
        self.calls = []

        class H(http.server.BaseHTTPRequestHandler):
            def _serve(self):
                n = int(self.headers.get("Content-Length") or 0)
                body = json.loads(self.rfile.read(n) or b"null") if n else None
                fake.calls.append((self.command, self.path, dict(self.headers), body))
                for (m, prefix), fn in routes.items():
                    if m == self.command and self.path.startswith(prefix):
                        status, payload = fn(self.path, dict(self.headers), body)
                        raw = json.dumps(payload).encode()
                        self.send_response(status)
                        self.send_header("Content-Type", "application/json")
                        self.send_header("Content-Length", str(len(raw)))
                        self.end_headers()
                        self.wfile.write(raw)
                        return
                self.send_response(404)
                self.send_header("Content-Length", "0")
                self.end_headers()
            do_GET = do_POST = _serve

            def log_message(self, *a):
                pass
        self.httpd = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
        self.url = f"http://127.0.0.1:{self.httpd.server_address[1]}"
        threading.Thread(target=self.httpd.serve_forever, daemon=True).start()

    def close(self):
        self.httpd.shutdown()
        self.httpd.server_close()


def test_secrets_manager_reads_vault_then_environment(monkeypatch):
    from axonml_b200.integrations.secrets import EnvBackend, SecretKey, SecretsError, SecretsManager, VaultBackend
    doc = {"jwt_secret": "from-vault-0123456789abcdef0123456789"}

    def read(path, headers, body):
        return (200, {"data": {"data": doc}}) if headers.get("X-Vault-Token") == "tok" else (403, {"errors": ["denied"]})

    def write(path, headers, body):
        doc.clear()
        doc.update(body["data"])
        return 200, {}
    fake = _Fake({("GET", "/v1/secret/data/axonml"): read, ("POST", "/v1/secret/data/axonml"): write,
                  ("POST", "/v1/auth/approle/login"): lambda p, h, b: (200, {"auth": {"client_token": "tok"}})})
    try:
        monkeypatch.setenv("AXONML_RESEND_API_KEY", "re_env")
        mgr = SecretsManager([VaultBackend(fake.url, "tok"), EnvBackend()])
        assert mgr.backend_names() == ["vault", "env"]
        assert mgr.get_secret(SecretKey.JWT_SECRET).startswith("from-vault")
        assert mgr.get_secret(SecretKey.RESEND_API_KEY) == "re_env"           # not in Vault: the next backend answers
        with pytest.raises(SecretsError, match="not found"):
            mgr.get_secret("db_password")
        approle = VaultBackend(fake.url, None, role_id="r", secret_id="s")       # AppRole login gets the token
        approle.put_secrets({"db_password": "pw"})
        assert VaultBackend(fake.url, "tok").get_secret("db_password") == "pw"
        with pytest.raises(SecretsError, match="refused"):
            VaultBackend(fake.url, "wrong").get_secret("jwt_secret")
        monkeypatch.setenv("VAULT_ADDR", fake.url)
        monkeypatch.setenv("VAULT_TOKEN", "tok")
        # the server signs its tokens with the secret from Vault
        srv = PlatformServer(port=0)
        try:
            assert srv.jwt.validate_access_token(JwtAuth(doc["jwt_secret"]).create_access_token("u", "e", "user")).sub == "u"
        finally:
            srv.httpd.server_close()
    finally:
        fake.close()


def test_registration_waits_for_the_mailed_verification_link(tmp_path):
    from axonml_b200.integrations.email import EmailService
    mails = []

    def send(path, headers, body):
        assert headers.get("Authorization") == "Bearer re_test"
        mails.append(body)
        return 200, {"id": f"mail-{len(mails)}"}
    fake = _Fake({("POST", "/emails"): send})
    srv = PlatformServer(port=0, data_dir=str(tmp_path / "srv"), allow_registration=True,
                         email=EmailService("re_test", base_url=fake.url)).start()
    try:
        c = Client(srv.port)
        assert c.req("POST", "/api/auth/register", {"email": "root@example.com", "name": "Root", "password": "s3cret-pass"})[0] == 201
        assert not mails                                                     # the first account (administrator) needs no link
        st, j = c.req("POST", "/api/auth/register", {"email": "eve@example.com", "name": "Eve", "password": "s3cret-pass"})
        assert st == 201 and j["user"]["email_verified"] is False and "inbox" in j["message"]
        assert [m["to"] for m in mails] == [["eve@example.com"], ["root@example.com"]]
        assert c.req("POST", "/api/auth/login", {"email": "eve@example.com", "password": "s3cret-pass"})[0] == 403
        link = mails[0]["html"].split('href="')[1].split('"')[0]
        assert link.startswith(srv.public_url + "/api/auth/verify-email?token=")
        assert c.req("GET", "/api/auth/verify-email?token=bogus")[0] == 400
        st, j = c.req("GET", link[len(srv.public_url):])
        assert st == 200 and j["user"]["email_verified"] and j["user"]["approved"]
        assert mails[-1]["subject"].startswith("Your AxonML account")          # welcome message
        assert c.req("GET", link[len(srv.public_url):])[0] == 400              # the link works once
        assert _login(c, "eve@example.com")["access_token"]
    finally:
        srv.stop()
        fake.close()


def test_notebook_ai_assist_asks_the_ollama_daemon(tmp_path):
    def gen(path, headers, body):
        assert body["stream"] is False and "Task: plot the loss" in body["prompt"] and "import torch" in body["prompt"]
        return 200, {"response": "Here you go:\n```python\nplt.plot(losses)\n```\n", "done": True}
    fake = _Fake({("GET", "/api/tags"): lambda p, h, b: (200, {"models": [{"name": "qwen2.5-coder:7b"}]}),
                  ("POST", "/api/generate"): gen})
    srv = PlatformServer(port=0, data_dir=str(tmp_path / "srv"), ollama_url=fake.url).start()
    try:
        c = Client(srv.port)
        c.req("POST", "/api/auth/register", {"email": "ada@example.com", "name": "Ada", "password": "s3cret-pass"})
        c.token = _login(c)["access_token"]
        nb = c.req("POST", "/api/notebooks", {"name": "n", "cells": [{"cell_type": "code", "source": "import torch"}]})[1]
        st, j = c.req("POST", f"/api/notebooks/{nb['id']}/ai-assist", {"prompt": "plot the loss"})
        assert st == 200 and j == {"kind": "code", "language": "python", "content": "plt.plot(losses)", "model": "qwen2.5-coder:7b"}
        from axonml_b200.integrations.ollama import OllamaClient
        assert OllamaClient(fake.url).list_models() == ["qwen2.5-coder:7b"]
        srv.ollama_url = "http://127.0.0.1:9"                                   # nothing listens there
        assert c.req("POST", f"/api/notebooks/{nb['id']}/ai-assist", {"prompt": "x"})[0] == 503
    finally:
        srv.stop()
        fake.close()
