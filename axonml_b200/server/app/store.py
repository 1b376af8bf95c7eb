"""Embedded document store for the platform server.

The reference server keeps users, runs, models, datasets and notebooks in an external Aegis-DB
document store reached over HTTP (crates/axonml-server/src/db/mod.rs:38-230: collections,
documents with ids, key/value entries, a query endpoint).  This build keeps the same three shapes
in one process: named collections of JSON documents, a key/value table and a small filter query,
all persisted to one JSON file per collection under a data directory with atomic replace, so a
server restart sees what the previous one wrote.  No network service is needed."""
from __future__ import annotations

import copy
import json
import os
import threading
import time
import uuid


class DbError(Exception):
    pass


class NotFound(DbError):
    pass


class AlreadyExists(DbError):
    pass


def now_iso() -> str:
    return time.strftime("%Y-%m-%dT%H:%M:%S", time.gmtime()) + "Z"


def _match(doc: dict, flt: dict) -> bool:
    """Equality on plain values; ``{"$gt"/"$gte"/"$lt"/"$lte"/"$ne"/"$in"/"$contains": v}`` on a field."""
    for k, want in flt.items():
        have = doc
        for part in k.split("."):
            have = have.get(part) if isinstance(have, dict) else None
        if isinstance(want, dict) and any(op.startswith("$") for op in want):
            for op, v in want.items():
                try:
                    ok = {"$gt": lambda: have > v, "$gte": lambda: have >= v, "$lt": lambda: have < v,
                          "$lte": lambda: have <= v, "$ne": lambda: have != v, "$in": lambda: have in v,
                          "$contains": lambda: v in (have or "")}[op]()
                except (TypeError, KeyError):
                    ok = False
                if not ok:
                    return False
        elif have != want:
            return False
    return True


class Collection:
    def __init__(self, store: "DocumentStore", name: str):
        self.store, self.name = store, name
        self._docs: dict[str, dict] = {}
        self._lock = threading.RLock()
        self._path = os.path.join(store.root, f"{name}.json") if store.root else None
        if self._path and os.path.exists(self._path):
            with open(self._path) as f:
                self._docs = json.load(f)

    def _flush(self) -> None:
        if not self._path:
            return
        tmp = self._path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self._docs, f)
        os.replace(tmp, self._path)

    # ------------------------------------------------------------------ documents
    def insert(self, doc: dict, doc_id: str | None = None) -> dict:
        with self._lock:
            doc = copy.deepcopy(doc)        # the store never shares mutable state with its callers
            doc_id = doc_id or doc.get("id") or uuid.uuid4().hex
            if doc_id in self._docs:
                raise AlreadyExists(f"{self.name}/{doc_id}")
            doc["id"] = doc_id
            doc.setdefault("created_at", now_iso())
            self._docs[doc_id] = doc
            self._flush()
            return copy.deepcopy(doc)

    def get(self, doc_id: str) -> dict:
        with self._lock:
            if doc_id not in self._docs:
                raise NotFound(f"{self.name}/{doc_id}")
            return copy.deepcopy(self._docs[doc_id])

    def find_one(self, **flt) -> dict | None:
        r = self.find(flt, limit=1)
        return r[0] if r else None

    def find(self, flt: dict | None = None, limit: int | None = None, offset: int = 0, sort: str | None = None,
             descending: bool = False) -> list[dict]:
        with self._lock:
            rows = [copy.deepcopy(d) for d in self._docs.values() if _match(d, flt or {})]
        if sort:
            rows.sort(key=lambda d: (d.get(sort) is None, d.get(sort)), reverse=descending)
        rows = rows[offset:]
        return rows[:limit] if limit is not None else rows

    def count(self, flt: dict | None = None) -> int:
        with self._lock:
            return sum(1 for d in self._docs.values() if _match(d, flt or {}))

    def update(self, doc_id: str, changes: dict) -> dict:
        with self._lock:
            if doc_id not in self._docs:
                raise NotFound(f"{self.name}/{doc_id}")
            self._docs[doc_id].update(copy.deepcopy({k: v for k, v in changes.items() if k != "id"}))
            self._docs[doc_id]["updated_at"] = now_iso()
            self._flush()
            return copy.deepcopy(self._docs[doc_id])

    def delete(self, doc_id: str) -> None:
        with self._lock:
            if doc_id not in self._docs:
                raise NotFound(f"{self.name}/{doc_id}")
            del self._docs[doc_id]
            self._flush()

    def delete_where(self, flt: dict) -> int:
        with self._lock:
            ids = [i for i, d in self._docs.items() if _match(d, flt)]
            for i in ids:
                del self._docs[i]
            if ids:
                self._flush()
            return len(ids)


class DocumentStore:
    """``root=None`` keeps everything in memory (tests)."""

    COLLECTIONS = ("users", "runs", "metrics", "logs", "models", "versions", "datasets", "endpoints", "notebooks",
                   "checkpoints", "kv")

    def __init__(self, root: str | None = None):
        self.root = root
        if root:
            os.makedirs(root, exist_ok=True)
        self._cols: dict[str, Collection] = {}
        self._lock = threading.Lock()

    def collection(self, name: str) -> Collection:
        with self._lock:
            if name not in self._cols:
                self._cols[name] = Collection(self, name)
            return self._cols[name]

    __getitem__ = collection

    # key/value table (the reference stores settings and counters this way)
    def kv_set(self, key: str, value) -> None:
        kv = self.collection("kv")
        try:
            kv.update(key, {"value": value})
        except NotFound:
            kv.insert({"value": value}, doc_id=key)

    def kv_get(self, key: str, default=None):
        try:
            return self.collection("kv").get(key)["value"]
        except NotFound:
            return default

    def query(self, collection: str, flt: dict | None = None, **kw) -> dict:
        """The admin query endpoint: rows + count, the reference's ``QueryResponse`` shape."""
        rows = self.collection(collection).find(flt, **kw)
        return {"rows": rows, "affected_rows": len(rows)}

    def health(self) -> dict:
        return {"status": "ok", "backend": "embedded", "persistent": bool(self.root),
                "collections": {n: c.count() for n, c in self._cols.items()}}
