"""The platform server: REST + WebSocket API over the document store, with authentication, training
runs, model registry, datasets, inference endpoints, system information, hub, notebooks, terminal
and the single-page dashboard.

Parity: the route table of crates/axonml-server/src/api/mod.rs:107-394 (public, authenticated and
admin groups; default port 3021).  The HTTP layer is the standard library's threaded
``http.server``; handlers are plain functions ``fn(req) -> (status, body)`` registered on a small
regex router, so every route can also be called in-process by tests through ``PlatformServer.call``."""
from __future__ import annotations

import json
import os
import re
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import parse_qs, urlparse

from ..inference import InferenceServer
from ..metrics import InferenceMetrics
from . import auth as A
from .notebooks import NotebookService
from .registry import DatasetCatalog, EndpointManager, ModelRegistry
from .store import AlreadyExists, DocumentStore, NotFound
from .system import SystemMonitor
from .training import RunRepository, TrainingExecutor, TrainingTracker


class HttpError(Exception):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status, self.message = status, message


class Request:
    def __init__(self, method: str, path: str, query: dict, headers, body: bytes, params: dict, app: "PlatformServer",
                 handler=None):
        self.method, self.path, self.query, self.headers, self.raw = method, path, query, headers, body
        self.params, self.app, self.handler = params, app, handler
        self.claims: A.Claims | None = None
        self._json = None

    @property
    def json(self) -> dict:
        if self._json is None:
            if not self.raw:
                self._json = {}
            else:
                try:
                    self._json = json.loads(self.raw)
                except ValueError:
                    raise HttpError(400, "request body is not valid JSON") from None
                if not isinstance(self._json, dict):
                    raise HttpError(400, "request body must be a JSON object")
        return self._json

    def need(self, *keys):
        missing = [k for k in keys if k not in self.json]
        if missing:
            raise HttpError(400, "missing field(s): " + ", ".join(missing))
        return [self.json[k] for k in keys]

    def q(self, key: str, default=None, cast=str):
        v = self.query.get(key)
        if not v:
            return default
        try:
            return cast(v[0])
        except ValueError:
            raise HttpError(400, f"bad query parameter {key}") from None

    @property
    def user_id(self) -> str:
        return self.claims.sub if self.claims else ""

    def upload(self) -> tuple[str, bytes, dict]:
        """(filename, bytes, other fields) of an upload sent as multipart/form-data, as JSON with a
        base64 ``data`` field, or as a raw body with ``?filename=``."""
        ctype = self.headers.get("Content-Type", "") if self.headers else ""
        if ctype.startswith("multipart/form-data"):
            from email.parser import BytesParser
            from email.policy import HTTP
            msg = BytesParser(policy=HTTP).parsebytes(b"Content-Type: " + ctype.encode() + b"\r\n\r\n" + self.raw)
            fields, fname, data = {}, "", b""
            for part in msg.iter_parts():
                name = part.get_param("name", header="content-disposition")
                if part.get_filename():
                    fname, data = part.get_filename(), part.get_payload(decode=True) or b""
                elif name:
                    fields[name] = (part.get_payload(decode=True) or b"").decode("utf-8", "replace")
            return fname, data, fields
        if ctype.startswith("application/json"):
            import base64
            j = dict(self.json)
            try:
                data = base64.b64decode(j.pop("data", ""))
            except ValueError:
                raise HttpError(400, "data must be base64") from None
            return j.pop("filename", "upload.bin"), data, j
        return self.q("filename", "upload.bin"), self.raw, {k: v[0] for k, v in self.query.items()}


PUBLIC, USER, ADMIN = "public", "user", "admin"


class Router:
    def __init__(self):
        self.routes: list = []

    def add(self, method: str, pattern: str, fn, access: str = USER) -> None:
        rx = re.compile("^" + re.sub(r":(\w+)", r"(?P<\1>[^/]+)", pattern) + "$")
        self.routes.append((method, rx, fn, access, pattern))

    def match(self, method: str, path: str):
        seen_path = False
        for m, rx, fn, access, _ in self.routes:
            mo = rx.match(path)
            if mo:
                seen_path = True
                if m == method:
                    return fn, access, mo.groupdict()
        if seen_path:
            raise HttpError(405, "method not allowed")
        raise HttpError(404, "not found")


class PlatformServer:
    def __init__(self, host: str = "127.0.0.1", port: int = 3021, data_dir: str | None = None, jwt_secret: str | None = None,
                 inference: InferenceServer | None = None, llm_engine=None, tokenizer=None, allow_registration: bool | None = None,
                 admin_email: str = "admin@axonml.local", admin_password: str | None = None,
                 enable_terminal: bool = False, secrets=None, email=None, ollama_url: str | None = None,
                 ollama_model: str | None = None, public_url: str | None = None):
        """``secrets``: an ``integrations.secrets.SecretsManager`` (default: Vault when ``VAULT_ADDR``
        is set, then ``AXONML_*`` environment variables) consulted for the JWT secret and the e-mail
        API key.  ``email``: an ``integrations.email.EmailService``; when it is configured, new
        accounts must confirm their address through a mailed link before they can sign in.
        ``ollama_url``: daemon behind the notebook AI assist.  ``public_url``: origin users reach
        the server at (links in e-mails, WebAuthn relying-party origin)."""
        from ...integrations.email import EmailService
        from ...integrations.secrets import SecretKey, SecretsManager
        self.data_dir = data_dir
        self.store = DocumentStore(os.path.join(data_dir, "db") if data_dir else None)
        files = os.path.join(data_dir, "files") if data_dir else os.path.join(_tmp_root(), "files")
        self.secrets = secrets if secrets is not None else SecretsManager.default()
        self.email = email if email is not None else EmailService(self.secrets.get_secret_optional(SecretKey.RESEND_API_KEY))
        self.ollama_url = ollama_url or os.environ.get("AXONML_OLLAMA_URL")
        self.ollama_model = ollama_model or os.environ.get("AXONML_OLLAMA_MODEL")
        secret = jwt_secret or self.secrets.get_secret_optional(SecretKey.JWT_SECRET) or self.store.kv_get("jwt_secret")
        if not secret:
            secret = os.urandom(32).hex()
            self.store.kv_set("jwt_secret", secret)
        self.jwt = A.JwtAuth(secret)
        self.totp = A.TotpAuth()
        self.users = self.store["users"]
        self.runs = RunRepository(self.store)
        self.tracker = TrainingTracker(self.runs)
        self.executor = TrainingExecutor(self.tracker, os.path.join(files, "runs"))
        self.registry = ModelRegistry(self.store, os.path.join(files, "models"))
        self.datasets = DatasetCatalog(self.store, os.path.join(files, "datasets"))
        self.inference = inference or InferenceServer()
        self.endpoints = EndpointManager(self.store, self.registry, self.inference)
        self.notebooks = NotebookService(self.store)
        self.monitor = SystemMonitor()
        self.metrics = InferenceMetrics()
        self.engine, self.tokenizer = llm_engine, tokenizer
        self.allow_registration, self.enable_terminal = allow_registration, enable_terminal
        self.revoked: set[str] = set()
        self.started = time.time()
        self.router = Router()
        from . import routes_assets, routes_auth, routes_misc, routes_tools, routes_training
        for mod in (routes_auth, routes_training, routes_tools, routes_assets, routes_misc):
            mod.register(self)
        if self.users.count() == 0 and admin_password:
            self.create_user(admin_email, "admin", admin_password, role="admin")
        self.httpd = ThreadingHTTPServer((host, port), _make_handler(self))
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        self.public_url = (public_url or f"http://localhost:{self.port}").rstrip("/")
        from urllib.parse import urlparse as _urlparse
        from .webauthn import WebAuthnAuth
        self.webauthn = WebAuthnAuth(_urlparse(self.public_url).hostname or "localhost", "AxonML", self.public_url)
        self._thread = None

    # ------------------------------------------------------------------ users
    def create_user(self, email: str, name: str, password: str, role: str = "user") -> dict:
        if role not in A.ROLES:
            raise HttpError(400, f"role must be one of {A.ROLES}")
        if self.users.find_one(email=email.lower()):
            raise AlreadyExists(f"user {email}")
        return self.users.insert({"email": email.lower(), "name": name, "password_hash": A.hash_password(password),
                                  "role": role, "mfa_enabled": False, "totp_secret": None, "pending_totp_secret": None,
                                  "recovery_codes": [], "webauthn_credentials": [], "email_verified": True,
                                  "approved": True, "last_login": None})

    @staticmethod
    def public_user(u: dict) -> dict:
        out = {k: u.get(k) for k in ("id", "email", "name", "role", "mfa_enabled", "email_verified", "approved",
                                     "created_at", "last_login")}
        out["webauthn_enabled"] = bool(u.get("webauthn_credentials"))
        return out

    # ------------------------------------------------------------------ dispatch
    def authenticate(self, req: Request, access: str) -> None:
        if access == PUBLIC:
            return
        tok = A.JwtAuth.extract_from_header(req.headers.get("Authorization") if req.headers else None) or req.q("token")
        if not tok:
            raise HttpError(401, "missing bearer token")
        if tok in self.revoked:
            raise HttpError(401, "token revoked")
        try:
            req.claims = self.jwt.validate_access_token(tok)
        except A.AuthError as e:
            raise HttpError(e.status, str(e)) from None
        if access == ADMIN and req.claims.role != "admin":
            raise HttpError(403, "administrator role required")

    def dispatch(self, req: Request):
        fn, access, params = self.router.match(req.method, req.path)
        req.params = params
        self.authenticate(req, access)
        return fn(req)

    def call(self, method: str, path: str, body=None, token: str | None = None, headers: dict | None = None):
        """In-process request (tests, CLI without a socket): returns (status, body)."""
        u = urlparse(path)
        raw = body if isinstance(body, bytes) else (json.dumps(body).encode() if body is not None else b"")
        h = dict(headers or {})
        if token:
            h["Authorization"] = "Bearer " + token
        if body is not None and not isinstance(body, bytes):
            h.setdefault("Content-Type", "application/json")
        req = Request(method, u.path, parse_qs(u.query), h, raw, {}, self)
        try:
            out = self.dispatch(req)
            return out if isinstance(out, tuple) else (200, out)
        except HttpError as e:
            return e.status, {"error": e.message}
        except NotFound as e:
            return 404, {"error": f"not found: {e}"}
        except AlreadyExists as e:
            return 409, {"error": f"already exists: {e}"}
        except A.AuthError as e:
            return e.status, {"error": str(e)}
        except PermissionError as e:                  # e.g. a service whose credentials are not configured
            return 403, {"error": str(e)}
        except (ValueError, KeyError) as e:
            return 400, {"error": f"{type(e).__name__}: {e}"}

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "PlatformServer":
        self._thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self._thread.start()
        return self

    def serve_forever(self) -> None:
        self.httpd.serve_forever()

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()
        self.notebooks.shutdown()


def _tmp_root() -> str:
    import tempfile
    return tempfile.mkdtemp(prefix="axonml_server_")


def _make_handler(app: PlatformServer):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):
            pass

        def _respond(self, status: int, body, ctype: str | None = None) -> None:
            if isinstance(body, (dict, list)) or body is None:
                data, ctype = json.dumps(body).encode(), ctype or "application/json"
            elif isinstance(body, str):
                data, ctype = body.encode(), ctype or "text/plain; charset=utf-8"
            else:
                data, ctype = bytes(body), ctype or "application/octet-stream"
            self.send_response(status)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            self.send_header("Access-Control-Allow-Origin", "*")
            self.end_headers()
            self.wfile.write(data)

        def _handle(self, method: str) -> None:
            u = urlparse(self.path)
            n = int(self.headers.get("Content-Length", 0) or 0)
            raw = self.rfile.read(n) if n else b""
            req = Request(method, u.path, parse_qs(u.query), self.headers, raw, {}, app, handler=self)
            t0 = time.perf_counter()
            try:
                out = app.dispatch(req)
                if out is None:                 # the route took over the socket (WebSocket)
                    return
                status, body = out if isinstance(out, tuple) and len(out) == 2 and isinstance(out[0], int) else (200, out)
                ctype = None
                if isinstance(body, tuple):     # (payload, content type)
                    body, ctype = body
                self._respond(status, body, ctype)
                ok = status < 400
            except HttpError as e:
                self._respond(e.status, {"error": e.message}); ok = False
            except NotFound as e:
                self._respond(404, {"error": f"not found: {e}"}); ok = False
            except AlreadyExists as e:
                self._respond(409, {"error": f"already exists: {e}"}); ok = False
            except A.AuthError as e:
                self._respond(e.status, {"error": str(e)}); ok = False
            except PermissionError as e:              # e.g. a service whose credentials are not configured
                self._respond(403, {"error": str(e)}); ok = False
            except (ValueError, KeyError) as e:
                self._respond(400, {"error": f"{type(e).__name__}: {e}"}); ok = False
            except Exception as e:  # noqa: BLE001 - the server must answer
                self._respond(500, {"error": f"{type(e).__name__}: {e}"}); ok = False
            if u.path.startswith("/api/inference/predict") or u.path == "/v1/completions":
                app.metrics.record(u.path, (time.perf_counter() - t0) * 1e3, ok)

        def do_GET(self): self._handle("GET")
        def do_POST(self): self._handle("POST")
        def do_PUT(self): self._handle("PUT")
        def do_DELETE(self): self._handle("DELETE")

        def do_OPTIONS(self):
            self.send_response(204)
            self.send_header("Access-Control-Allow-Origin", "*")
            self.send_header("Access-Control-Allow-Methods", "GET, POST, PUT, DELETE, OPTIONS")
            self.send_header("Access-Control-Allow-Headers", "Authorization, Content-Type")
            self.send_header("Content-Length", "0")
            self.end_headers()

    return Handler
