"""Secrets for the platform server: a manager that asks its backends in order
(crates/axonml-server/src/secrets/mod.rs:43-140), an environment backend
(``AXONML_<KEY>``, secrets/env.rs) and a HashiCorp Vault KV v2 backend over its HTTP API
(secrets/vault.rs: token or AppRole login, mount and path from the environment)."""
from __future__ import annotations

import json
import os
import urllib.error
import urllib.request


class SecretsError(RuntimeError):
    pass


class SecretKey:
    JWT_SECRET = "jwt_secret"
    DB_USERNAME = "db_username"
    DB_PASSWORD = "db_password"
    RESEND_API_KEY = "resend_api_key"


class EnvBackend:
    name = "env"

    def __init__(self, prefix: str = "AXONML_"):
        self.prefix = prefix

    def get_secret(self, key: str):
        return os.environ.get(self.prefix + key.upper()) or None


class VaultBackend:
    """KV version 2 secrets under ``<mount>/data/<path>``; one document holds all keys."""
    name = "vault"

    def __init__(self, addr: str, token: str | None = None, mount: str = "secret", path: str = "axonml",
                 role_id: str | None = None, secret_id: str | None = None, timeout: float = 5.0):
        self.addr, self.mount, self.path, self.timeout = addr.rstrip("/"), mount.strip("/"), path.strip("/"), timeout
        self.token = token
        self._cache: dict | None = None
        if token is None:
            if not (role_id and secret_id):
                raise SecretsError("Vault needs a token or an AppRole role id and secret id")
            out = self._call("POST", "/v1/auth/approle/login", {"role_id": role_id, "secret_id": secret_id}, auth=False)
            try:
                self.token = out["auth"]["client_token"]
            except (KeyError, TypeError) as e:
                raise SecretsError("AppRole login returned no token") from e

    @classmethod
    def from_env(cls):
        """``VAULT_ADDR`` with ``VAULT_TOKEN`` or ``VAULT_ROLE_ID`` + ``VAULT_SECRET_ID``
        (``VAULT_MOUNT``, ``VAULT_PATH`` optional); None when no address is set."""
        addr = os.environ.get("VAULT_ADDR")
        if not addr:
            return None
        return cls(addr, os.environ.get("VAULT_TOKEN"), os.environ.get("VAULT_MOUNT", "secret"),
                   os.environ.get("VAULT_PATH", "axonml"), os.environ.get("VAULT_ROLE_ID"), os.environ.get("VAULT_SECRET_ID"))

    def _call(self, method: str, route: str, body: dict | None = None, auth: bool = True):
        req = urllib.request.Request(self.addr + route, method=method,
                                     data=None if body is None else json.dumps(body).encode())
        req.add_header("Content-Type", "application/json")
        if auth and self.token:
            req.add_header("X-Vault-Token", self.token)
        try:
            with urllib.request.urlopen(req, timeout=self.timeout) as r:
                raw = r.read()
        except urllib.error.HTTPError as e:
            if e.code == 404:
                return None
            if e.code in (401, 403):
                raise SecretsError(f"Vault refused the request ({e.code})") from e
            raise SecretsError(f"Vault error {e.code}") from e
        except (urllib.error.URLError, OSError) as e:
            raise SecretsError(f"Vault is unreachable: {e}") from e
        return json.loads(raw) if raw else {}

    def _document(self) -> dict:
        if self._cache is None:
            out = self._call("GET", f"/v1/{self.mount}/data/{self.path}")
            self._cache = ((out or {}).get("data") or {}).get("data") or {}
        return self._cache

    def get_secret(self, key: str):
        v = self._document().get(key)
        return None if v is None else str(v)

    def put_secrets(self, values: dict) -> None:
        doc = dict(self._document())
        doc.update(values)
        self._call("POST", f"/v1/{self.mount}/data/{self.path}", {"data": doc})
        self._cache = doc

    def renew_token(self) -> bool:
        return self._call("POST", "/v1/auth/token/renew-self", {}) is not None


class SecretsManager:
    def __init__(self, backends: list | None = None):
        self.backends = list(backends or [])

    @classmethod
    def default(cls):
        """Vault first when ``VAULT_ADDR`` is set, then the environment."""
        backends = []
        try:
            v = VaultBackend.from_env()
            if v is not None:
                backends.append(v)
        except SecretsError:
            pass
        backends.append(EnvBackend())
        return cls(backends)

    def with_backend(self, backend) -> "SecretsManager":
        self.backends.append(backend)
        return self

    def get_secret_optional(self, key: str):
        for b in self.backends:
            v = b.get_secret(key)
            if v:
                return v
        return None

    def get_secret(self, key: str) -> str:
        v = self.get_secret_optional(key)
        if v is None:
            raise SecretsError(f"secret not found: {key}")
        return v

    def has_backends(self) -> bool:
        return bool(self.backends)

    def backend_names(self) -> list:
        return [b.name for b in self.backends]
