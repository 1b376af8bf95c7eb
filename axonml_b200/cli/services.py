"""Service and integration commands of the CLI: ``start`` / ``stop`` / ``status`` / ``logs`` for the
platform server, ``login`` / ``logout`` / ``sync`` against a running server, ``wandb``, ``kaggle``,
``dataset`` and ``tui``.

Parity: crates/axonml-cli/src/commands/{dashboard,sync,wandb,kaggle,dataset,tui}.rs and their
argument structs (cli.rs:500-566, 1411-1715).  The reference starts two processes (API server and
a dashboard dev server); here one process serves the API and the dashboard page, so ``--server``
and ``--dashboard`` select the same process.  State (pid file, log file, session token) lives under
``$AXONML_HOME`` (default ``~/.axonml``)."""
from __future__ import annotations

import getpass
import json
import os
import signal
import subprocess
import sys
import time
import urllib.error
import urllib.request


def home() -> str:
    d = os.environ.get("AXONML_HOME") or os.path.join(os.path.expanduser("~"), ".axonml")
    os.makedirs(d, exist_ok=True)
    return d


def _pid_file() -> str: return os.path.join(home(), "server.pid")
def _log_file() -> str: return os.path.join(home(), "server.log")
def _session_file() -> str: return os.path.join(home(), "session.json")


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except (OSError, ProcessLookupError):
        return False


def _read_pid() -> dict | None:
    try:
        with open(_pid_file()) as f:
            d = json.load(f)
        return d if _alive(int(d["pid"])) else None
    except (OSError, ValueError, KeyError):
        return None


# ----------------------------------------------------------------------------- start / stop / status / logs
def cmd_start(a) -> None:
    cur = _read_pid()
    if cur:
        raise SystemExit(f"already running: pid {cur['pid']} on http://{cur['host']}:{cur['port']}")
    data_dir = os.path.join(home(), "server")
    if a.foreground:
        from ..server.app import PlatformServer
        srv = PlatformServer(a.host, a.port, data_dir, admin_password=os.environ.get("AXONML_ADMIN_PASSWORD"),
                             enable_terminal=bool(os.environ.get("AXONML_ENABLE_TERMINAL")))
        with open(_pid_file(), "w") as f:
            json.dump({"pid": os.getpid(), "host": a.host, "port": srv.port, "started": time.time()}, f)
        print(f"AxonML server and dashboard on http://{a.host}:{srv.port}", flush=True)
        try:
            srv.serve_forever()
        except KeyboardInterrupt:
            pass
        finally:
            if os.path.exists(_pid_file()):
                os.remove(_pid_file())
        return
    log = open(_log_file(), "a")
    cmd = [sys.executable, "-m", "axonml_b200.cli", "start", "--foreground", "--host", a.host, "--port", str(a.port)]
    pkg_parent = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env = dict(os.environ)
    env["PYTHONPATH"] = pkg_parent + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    proc = subprocess.Popen(cmd, stdout=log, stderr=log, stdin=subprocess.DEVNULL, start_new_session=True, env=env)
    for _ in range(900):                         # the first import of torch in a new process can take a minute
        time.sleep(0.1)
        cur = _read_pid()
        if cur and cur["pid"] == proc.pid:
            print(f"started pid {proc.pid}: http://{cur['host']}:{cur['port']}  (log: {_log_file()})")
            return
        if proc.poll() is not None:
            break
    raise SystemExit(f"the server did not come up; see {_log_file()}")


def cmd_stop(a) -> None:
    cur = _read_pid()
    if not cur:
        print("not running")
        return
    os.kill(int(cur["pid"]), signal.SIGKILL if a.force else signal.SIGTERM)      # the exact pid this CLI started
    for _ in range(50):
        if not _alive(int(cur["pid"])):
            break
        time.sleep(0.1)
    if os.path.exists(_pid_file()):
        os.remove(_pid_file())
    print(f"stopped pid {cur['pid']}")


def _http(method: str, url: str, body=None, token: str | None = None, timeout: float = 5.0):
    data = json.dumps(body).encode() if body is not None else None
    r = urllib.request.Request(url, data=data, method=method)
    if data is not None:
        r.add_header("Content-Type", "application/json")
    if token:
        r.add_header("Authorization", "Bearer " + token)
    try:
        with urllib.request.urlopen(r, timeout=timeout) as resp:
            return resp.status, json.loads(resp.read() or b"null")
    except urllib.error.HTTPError as e:
        try:
            return e.code, json.loads(e.read() or b"null")
        except ValueError:
            return e.code, None
    except (urllib.error.URLError, OSError) as e:
        return 0, {"error": str(getattr(e, "reason", e))}


def cmd_status(a) -> None:
    cur = _read_pid()
    st = {"running": bool(cur)}
    if cur:
        st.update(cur)
        code, h = _http("GET", f"http://{cur['host']}:{cur['port']}/health")
        st["healthy"] = code == 200
        if a.detailed and code == 200:
            st["health"] = h
            st["inference"] = _http("GET", f"http://{cur['host']}:{cur['port']}/api/status/inference")[1]
    if a.format == "json":
        print(json.dumps(st, indent=1))
    else:
        print("AxonML server: " + (f"running (pid {st['pid']}, http://{st['host']}:{st['port']}, "
                                   f"{'healthy' if st.get('healthy') else 'not answering'})" if cur else "stopped"))
        if a.detailed and cur:
            print(json.dumps({k: st[k] for k in ("health", "inference") if k in st}, indent=1))


def cmd_logs(a) -> None:
    path = _log_file()
    if not os.path.exists(path):
        print("no log yet")
        return

    def keep(line: str) -> bool:
        return not a.level or a.level.lower() in line.lower()

    with open(path) as f:
        lines = [l for l in f.readlines() if keep(l)]
        for l in lines[-a.lines:]:
            print(l, end="")
        if a.follow:
            try:
                while True:
                    l = f.readline()
                    if not l:
                        time.sleep(0.25)
                    elif keep(l):
                        print(l, end="", flush=True)
            except KeyboardInterrupt:
                pass


# ----------------------------------------------------------------------------- login / logout / sync
def _session() -> dict | None:
    try:
        with open(_session_file()) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


def cmd_login(a) -> None:
    a.username = getattr(a, "username_opt", None) or a.username or os.environ.get("AXONML_USER") or input("user (e-mail): ")
    server = (a.server or "http://localhost:3021").rstrip("/")
    password = a.password or os.environ.get("AXONML_PASSWORD") or getpass.getpass("password: ")
    code, j = _http("POST", server + "/api/auth/login", {"email": a.username, "password": password})
    if code == 200 and j.get("requires_mfa"):
        otp = os.environ.get("AXONML_OTP") or input("authenticator code: ")
        code, j = _http("POST", server + "/api/auth/mfa/totp/verify", {"mfa_token": j["mfa_token"], "code": otp})
    if code != 200:
        raise SystemExit(f"login failed: {(j or {}).get('error', code)}")
    fd = os.open(_session_file(), os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
    with os.fdopen(fd, "w") as f:
        json.dump({"server": server, "access_token": j["access_token"], "refresh_token": j["refresh_token"],
                   "user": j["user"]}, f)
    print(f"logged in to {server} as {j['user']['email']} ({j['user']['role']})")


def cmd_logout(a) -> None:
    s = _session()
    if s:
        _http("POST", s["server"] + "/api/auth/logout", token=s["access_token"])
        os.remove(_session_file())
    print("logged out")


def cmd_sync(a) -> None:
    """Compares local artefacts (./models, ./output checkpoints) with the server's registry and
    uploads what is missing; ``--check`` only reports."""
    s = _session()
    if not s:
        raise SystemExit("not logged in (axonml login <user>)")
    code, remote = _http("GET", s["server"] + "/api/models", token=s["access_token"])
    if code == 401 and s.get("refresh_token"):
        c2, pair = _http("POST", s["server"] + "/api/auth/refresh", {"refresh_token": s["refresh_token"]})
        if c2 == 200:
            s.update({"access_token": pair["access_token"], "refresh_token": pair["refresh_token"]})
            with open(_session_file(), "w") as f:
                json.dump(s, f)
            code, remote = _http("GET", s["server"] + "/api/models", token=s["access_token"])
    if code != 200:
        raise SystemExit(f"cannot reach {s['server']}: {(remote or {}).get('error', code)}")
    remote_names = {m["name"]: m for m in remote}
    local = []
    for d in ("models", "output"):
        if os.path.isdir(d):
            local += [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith((".axonml", ".safetensors", ".gguf", ".onnx"))]
    missing = [p for p in local if os.path.splitext(os.path.basename(p))[0] not in remote_names or a.force]
    print(f"server {s['server']}: {len(remote)} models; local: {len(local)} files; to upload: {len(missing)}")
    if a.check:
        for p in missing:
            print("  would upload", p)
        return
    import base64
    for p in missing:
        name = os.path.splitext(os.path.basename(p))[0]
        m = remote_names.get(name)
        if m is None:
            code, m = _http("POST", s["server"] + "/api/models", {"name": name}, s["access_token"])
            if code != 201:
                print(f"  {name}: create failed ({(m or {}).get('error', code)})")
                continue
        with open(p, "rb") as f:
            blob = base64.b64encode(f.read()).decode()
        code, v = _http("POST", f"{s['server']}/api/models/{m['id']}/versions", {"filename": os.path.basename(p), "data": blob},
                        s["access_token"], timeout=120)
        print(f"  {name}: " + (f"uploaded as version {v['version']}" if code == 201 else f"upload failed ({code})"))


# ----------------------------------------------------------------------------- wandb / kaggle / dataset
def cmd_wandb(a) -> None:
    from ..integrations.wandb import WandbConfig
    cfg = WandbConfig.load()
    act = a.action
    if act == "login":
        key = os.environ.get("WANDB_API_KEY") or getpass.getpass("W&B API key: ")
        if len(key) < 20:
            raise SystemExit("that does not look like a W&B API key")
        cfg.api_key = key
        print(f"saved to {cfg.save()}")
    elif act == "logout":
        cfg.api_key = None
        cfg.save()
        print("logged out of W&B")
    elif act == "status":
        for k, v in cfg.status().items():
            print(f"{k:16s} {v}")
    elif act == "config":
        for k in ("api_key", "entity", "project", "base_url", "log_frequency"):
            v = getattr(a, k, None)
            if v is not None:
                setattr(cfg, k, v)
        if a.log_checkpoints is not None:
            cfg.log_checkpoints = a.log_checkpoints
        if a.log_system is not None:
            cfg.log_system = a.log_system
        print(f"saved to {cfg.save()}")
    elif act in ("enable", "disable"):
        cfg.enabled = act == "enable"
        cfg.save()
        print(f"W&B logging {'enabled' if cfg.enabled else 'disabled'} (runs are written in offline layout under ./wandb)")


def cmd_kaggle(a) -> None:
    from ..integrations.kaggle import KaggleClient, OfflineError
    k = KaggleClient()
    try:
        if a.action == "login":
            a.username = getattr(a, "username_opt", None) or a.username or os.environ.get("KAGGLE_USERNAME") or input("Kaggle user name: ")
            key = a.key or os.environ.get("KAGGLE_KEY") or getpass.getpass("Kaggle API key: ")
            print(f"saved to {k.save_credentials(a.username, key)}")
        elif a.action == "status":
            for key, v in k.status().items():
                print(f"{key:12s} {v}")
        elif a.action == "search":
            for d in k.search(a.query, a.limit):
                print(f"{d['ref']:48s} {d['title']}")
        elif a.action == "download":
            r = k.download(a.dataset, a.output)
            print(f"downloaded {r['ref']} -> {r['path']} ({len(r['files'])} files)")
        elif a.action == "list":
            for d in k.list_downloaded():
                print(f"{d['ref']:48s} {d['files']:5d} files {d['bytes']:>14,} bytes  {d['path']}")
    except OfflineError as e:
        raise SystemExit(f"offline: {e}") from None
    except PermissionError as e:
        raise SystemExit(str(e)) from None


def cmd_dataset(a) -> None:
    from ..data import catalog as C
    if a.action == "list":
        for d in C.list_datasets(a.source):
            print(f"{d['id']:16s} {d['name']:30s} {d['type']:8s} {d['samples']:>7} samples  [{d['source']}]")
    elif a.action == "info":
        d = C.get_dataset_info(a.id)
        if d is None:
            raise SystemExit(f"unknown dataset {a.id!r}")
        for k, v in d.items():
            print(f"{k:10s} {v}")
    elif a.action == "search":
        hits = C.search_datasets(a.query, a.source, a.limit)
        for d in hits:
            print(f"{d['id']:16s} {d['name']:30s} [{d['source']}]")
        if not hits:
            print("no match in the built-in catalogue (remote sources need network access)")
    elif a.action == "sources":
        for s in C.SOURCES:
            print(f"{s['id']:10s} {s['name']:20s} {s['description']}")
    elif a.action == "download":
        d = C.get_dataset_info(a.id)
        if d is None:
            raise SystemExit(f"unknown dataset {a.id!r}")
        out = a.output or os.path.join("datasets", d["id"])
        if d.get("synthetic") and d["type"] == "image":
            # no route to the mirrors from this host: write the synthetic stand-in in the original
            # IDX file format, so that the real loader reads it
            from ..vision.datasets import write_synthetic_idx
            n = write_synthetic_idx(out, d["shape"], d["classes"], samples=2048)
            print(f"no network: wrote a synthetic stand-in of {d['id']} ({n} samples, IDX format) to {out}")
        else:
            raise SystemExit(f"{d['id']} has to be fetched from {d['source']}, which needs network access")


# ----------------------------------------------------------------------------- parser wiring
def add_parsers(sub) -> None:
    p = sub.add_parser("start", help="start the API server and dashboard")
    p.add_argument("--server", action="store_true"); p.add_argument("--dashboard", action="store_true")
    p.add_argument("--port", type=int, default=3021); p.add_argument("--dashboard-port", type=int, default=8080)
    p.add_argument("--host", default="127.0.0.1"); p.add_argument("-f", "--foreground", action="store_true"); p.add_argument("-c", "--config")
    p.set_defaults(fn=cmd_start)
    p = sub.add_parser("stop"); p.add_argument("--server", action="store_true"); p.add_argument("--dashboard", action="store_true")
    p.add_argument("-f", "--force", action="store_true"); p.set_defaults(fn=cmd_stop)
    p = sub.add_parser("status"); p.add_argument("-d", "--detailed", action="store_true")
    p.add_argument("-f", "--format", default="text", choices=["text", "json"]); p.set_defaults(fn=cmd_status)
    p = sub.add_parser("logs"); p.add_argument("--server", action="store_true"); p.add_argument("--dashboard", action="store_true")
    p.add_argument("--lines", "-n", "-l", type=int, default=50); p.add_argument("--follow", "-f", action="store_true"); p.add_argument("--level")
    p.set_defaults(fn=cmd_logs)
    p = sub.add_parser("login"); p.add_argument("username", nargs="?"); p.add_argument("-u", "--username", dest="username_opt")
    p.add_argument("-p", "--password"); p.add_argument("-s", "--server")
    p.set_defaults(fn=cmd_login)
    p = sub.add_parser("logout"); p.set_defaults(fn=cmd_logout)
    p = sub.add_parser("sync"); p.add_argument("--status", "--check", dest="check", action="store_true"); p.add_argument("--force", action="store_true")
    p.set_defaults(fn=cmd_sync)

    p = sub.add_parser("wandb", help="Weights & Biases settings")
    s = p.add_subparsers(dest="action", required=True)
    for name in ("login", "logout", "status", "enable", "disable"):
        s.add_parser(name)
    q = s.add_parser("config"); q.add_argument("--api-key", dest="api_key"); q.add_argument("-e", "--entity"); q.add_argument("-p", "--project")
    q.add_argument("--base-url", dest="base_url"); q.add_argument("--log-frequency", dest="log_frequency", type=int)
    q.add_argument("--log-checkpoints", dest="log_checkpoints", type=lambda v: v.lower() in ("1", "true", "yes"), default=None)
    q.add_argument("--log-system-metrics", "--log-system", dest="log_system", type=lambda v: v.lower() in ("1", "true", "yes"), default=None)
    p.set_defaults(fn=cmd_wandb)

    p = sub.add_parser("kaggle", help="Kaggle datasets")
    s = p.add_subparsers(dest="action", required=True)
    q = s.add_parser("login"); q.add_argument("username", nargs="?"); q.add_argument("-u", "--username", dest="username_opt"); q.add_argument("-k", "--key")
    s.add_parser("status"); s.add_parser("list")
    q = s.add_parser("search"); q.add_argument("query"); q.add_argument("-l", "--limit", type=int, default=10)
    q = s.add_parser("download"); q.add_argument("dataset"); q.add_argument("-o", "--output")
    p.set_defaults(fn=cmd_kaggle)

    p = sub.add_parser("dataset", help="dataset catalogue")
    s = p.add_subparsers(dest="action", required=True)
    q = s.add_parser("list"); q.add_argument("-s", "--source")
    q = s.add_parser("info"); q.add_argument("id")
    q = s.add_parser("search"); q.add_argument("query"); q.add_argument("-s", "--source"); q.add_argument("-l", "--limit", type=int, default=10)
    q = s.add_parser("download"); q.add_argument("id"); q.add_argument("-o", "--output")
    s.add_parser("sources")
    p.set_defaults(fn=cmd_dataset)

    from . import tui
    p = sub.add_parser("tui", help="terminal user interface")
    p.add_argument("-m", "--model"); p.add_argument("-d", "--data")
    p.add_argument("--watch", help="training log (JSON lines) to follow in the Training and Graphs views")
    p.add_argument("--once", action="store_true", help="render every view once and exit")
    p.set_defaults(fn=tui.cmd_tui)
