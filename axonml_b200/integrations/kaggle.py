"""Kaggle dataset client (crates/axonml-cli/src/commands/kaggle.rs, crates/axonml-server/src/api/kaggle.rs):
credentials in ``kaggle.json`` (mode 0600), status, search, download with unzip, and the list of
downloaded datasets.  The HTTP transport is ``urllib``; when the host has no route to
``www.kaggle.com`` the calls raise ``OfflineError`` instead of hanging (5 s timeout)."""
from __future__ import annotations

import base64
import json
import os
import urllib.error
import urllib.parse
import urllib.request
import zipfile

API = "https://www.kaggle.com/api/v1"


class OfflineError(RuntimeError):
    pass


class KaggleClient:
    def __init__(self, config_dir: str | None = None, data_dir: str | None = None, timeout: float = 5.0):
        self.config_dir = config_dir or os.environ.get("KAGGLE_CONFIG_DIR") or os.path.join(os.path.expanduser("~"), ".kaggle")
        self.data_dir = data_dir or os.path.join(self.config_dir, "datasets")
        self.timeout = timeout

    # ------------------------------------------------------------------ credentials
    @property
    def _cred_path(self) -> str:
        return os.path.join(self.config_dir, "kaggle.json")

    def save_credentials(self, username: str, key: str) -> str:
        os.makedirs(self.config_dir, exist_ok=True)
        fd = os.open(self._cred_path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
        with os.fdopen(fd, "w") as f:
            json.dump({"username": username, "key": key}, f)
        return self._cred_path

    def delete_credentials(self) -> None:
        if os.path.exists(self._cred_path):
            os.remove(self._cred_path)

    def credentials(self) -> dict | None:
        if os.environ.get("KAGGLE_USERNAME") and os.environ.get("KAGGLE_KEY"):
            return {"username": os.environ["KAGGLE_USERNAME"], "key": os.environ["KAGGLE_KEY"]}
        try:
            with open(self._cred_path) as f:
                return json.load(f)
        except (OSError, ValueError):
            return None

    def status(self) -> dict:
        c = self.credentials()
        return {"configured": c is not None, "username": c["username"] if c else None, "config_path": self._cred_path,
                "downloaded": len(self.list_downloaded())}

    # ------------------------------------------------------------------ transport
    def _request(self, path: str):
        c = self.credentials()
        if c is None:
            raise PermissionError("Kaggle credentials are not configured (axonml kaggle login)")
        req = urllib.request.Request(API + path)
        req.add_header("Authorization", "Basic " + base64.b64encode(f"{c['username']}:{c['key']}".encode()).decode())
        try:
            return urllib.request.urlopen(req, timeout=self.timeout)
        except (urllib.error.URLError, OSError, TimeoutError) as e:
            raise OfflineError(f"cannot reach www.kaggle.com: {getattr(e, 'reason', e)}") from None

    def search(self, query: str, limit: int = 10) -> list[dict]:
        with self._request("/datasets/list?search=" + urllib.parse.quote(query)) as r:
            rows = json.load(r)
        return [{"ref": d.get("ref"), "title": d.get("title"), "size": d.get("totalBytes"),
                 "downloads": d.get("downloadCount"), "votes": d.get("voteCount")} for d in rows[:limit]]

    def download(self, ref: str, output_dir: str | None = None) -> dict:
        if ref.count("/") != 1:
            raise ValueError("dataset reference must look like owner/dataset-name")
        out = output_dir or os.path.join(self.data_dir, ref.replace("/", "__"))
        os.makedirs(out, exist_ok=True)
        zpath = os.path.join(out, "dataset.zip")
        with self._request("/datasets/download/" + ref) as r, open(zpath, "wb") as f:
            while True:
                chunk = r.read(1 << 20)
                if not chunk:
                    break
                f.write(chunk)
        with zipfile.ZipFile(zpath) as z:
            z.extractall(out)
            names = z.namelist()
        os.remove(zpath)
        return {"ref": ref, "path": out, "files": names}

    def list_downloaded(self) -> list[dict]:
        if not os.path.isdir(self.data_dir):
            return []
        out = []
        for d in sorted(os.listdir(self.data_dir)):
            p = os.path.join(self.data_dir, d)
            if os.path.isdir(p):
                files = [os.path.join(r, f) for r, _, fs in os.walk(p) for f in fs]
                out.append({"ref": d.replace("__", "/"), "path": p, "files": len(files),
                            "bytes": sum(os.path.getsize(f) for f in files)})
        return out
