"""Weight download and cache shared by the vision and language-model hubs.

Parity: crates/axonml-vision/src/hub.rs:21-72, :94-100, :435-511 and crates/axonml-llm/src/hub.rs:
39-112, :594-673 (``HubError`` with its four kinds, a cache directory per hub, ``is_cached`` /
``cached_path``, ``download_weights(name, force)`` which returns the cached file unless forced).
Here the transfer goes to a temporary file that is renamed into place once complete (an
interrupted download leaves no half-written cache entry), an entry's SHA-256 is checked when the
registry gives one, and the host of every URL can be redirected with ``AXONML_HUB_ENDPOINT`` (a
mirror, or a local server in the tests)."""
from __future__ import annotations

import hashlib
import os
import urllib.error
import urllib.request

DEFAULT_ENDPOINT = "https://huggingface.co"


class HubError(Exception):
    """Base of the hub errors; ``kind`` is the reference's variant name."""
    kind = "HubError"


class NetworkError(HubError):
    kind = "NetworkError"

    def __str__(self) -> str: return "Network error: " + super().__str__()


class HubIoError(HubError):
    kind = "IoError"

    def __str__(self) -> str: return "IO error: " + super().__str__()


class ModelNotFound(HubError, KeyError):
    kind = "ModelNotFound"

    def __str__(self) -> str: return "Model not found: " + (self.args[0] if self.args else "")


class InvalidFormat(HubError, ValueError):
    kind = "InvalidFormat"

    def __str__(self) -> str: return "Invalid format: " + super().__str__()


def endpoint() -> str:
    return os.environ.get("AXONML_HUB_ENDPOINT", DEFAULT_ENDPOINT).rstrip("/")


def repo_url(repo: str, filename: str, revision: str = "main") -> str:
    """``<endpoint>/<org>/<repo>/resolve/<revision>/<file>``."""
    return f"{endpoint()}/{repo}/resolve/{revision}/{filename}"


def hub_cache_root() -> str:
    """``$AXONML_HUB_CACHE``, else ``$XDG_CACHE_HOME/axonml/hub``, else ``~/.cache/axonml/hub``."""
    root = os.environ.get("AXONML_HUB_CACHE")
    if not root:
        base = os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache")
        root = os.path.join(base, "axonml", "hub")
    return root


def format_params(n: int) -> str:
    for unit, div in (("B", 1e9), ("M", 1e6), ("K", 1e3)):
        if n >= div:
            return f"{n / div:.1f}{unit}"
    return str(n)


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def fetch(url: str, dest: str, checksum: str | None = None, timeout: float = 30.0, progress=None) -> str:
    """Downloads ``url`` to ``dest`` (through ``dest + '.part'``); raises ``NetworkError`` on a
    transport or HTTP failure and ``InvalidFormat`` when the SHA-256 differs from ``checksum``."""
    try:
        os.makedirs(os.path.dirname(dest) or ".", exist_ok=True)
    except OSError as e:
        raise HubIoError(str(e)) from e
    part = dest + ".part"
    try:
        req = urllib.request.Request(url, headers={"User-Agent": "axonml-hub"})
        with urllib.request.urlopen(req, timeout=timeout) as r:
            if getattr(r, "status", 200) != 200:
                raise NetworkError(f"HTTP {r.status}: {url}")
            total = int(r.headers.get("Content-Length") or 0)
            done = 0
            with open(part, "wb") as f:
                for chunk in iter(lambda: r.read(1 << 20), b""):
                    f.write(chunk)
                    done += len(chunk)
                    if progress:
                        progress(done, total)
    except urllib.error.HTTPError as e:
        _discard(part)
        raise NetworkError(f"HTTP {e.code}: {url}") from e
    except (urllib.error.URLError, TimeoutError, ConnectionError) as e:
        _discard(part)
        raise NetworkError(f"{getattr(e, 'reason', e)}: {url}") from e
    except OSError as e:
        _discard(part)
        raise HubIoError(str(e)) from e
    if checksum and sha256_file(part).lower() != checksum.lower():
        _discard(part)
        raise InvalidFormat(f"SHA-256 of {url} does not match the registry entry")
    os.replace(part, dest)
    return dest


def _discard(path: str) -> None:
    try:
        os.remove(path)
    except OSError:
        pass
