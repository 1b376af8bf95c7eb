"""Dataset inspection: type detection, statistics, preview, validation and a recommended training
configuration, for the ``data`` / ``analyze`` commands and the server's ``/api/data/*`` routes.

Parity: crates/axonml-cli/src/commands/data.rs (upload / analyze / list / config / preview /
validate: image-folder, tabular CSV, text, audio and IDX detection; class counts, imbalance ratio,
missing values, recommended batch size / learning rate / architecture) and
crates/axonml-server/src/api/data.rs."""
from __future__ import annotations

import csv
import json
import math
import os
import struct

IMAGE_EXT = {".png", ".jpg", ".jpeg", ".bmp", ".gif", ".ppm", ".pgm", ".webp"}
AUDIO_EXT = {".wav", ".flac", ".mp3", ".ogg"}
TEXT_EXT = {".txt", ".jsonl", ".md"}
TABULAR_EXT = {".csv", ".tsv", ".parquet"}


def detect_type(path: str) -> str:
    if os.path.isfile(path):
        ext = os.path.splitext(path)[1].lower()
        if ext in TABULAR_EXT:
            return "tabular"
        if ext in TEXT_EXT:
            return "text"
        if ext in AUDIO_EXT:
            return "audio"
        if ext in IMAGE_EXT:
            return "image"
        if "idx" in os.path.basename(path).lower():
            return "idx"
        return "unknown"
    counts = {"image": 0, "audio": 0, "text": 0, "tabular": 0, "idx": 0}
    for _, _, files in os.walk(path):
        for f in files:
            ext = os.path.splitext(f)[1].lower()
            for kind, exts in (("image", IMAGE_EXT), ("audio", AUDIO_EXT), ("text", TEXT_EXT), ("tabular", TABULAR_EXT)):
                if ext in exts:
                    counts[kind] += 1
            if "idx" in f.lower() and "ubyte" in f.lower():
                counts["idx"] += 1
    best = max(counts, key=counts.get)
    return best if counts[best] else "unknown"


def _idx_header(path: str) -> dict:
    import gzip
    op = gzip.open if path.endswith(".gz") else open
    with op(path, "rb") as f:
        magic = f.read(4)
        if len(magic) < 4 or magic[0] != 0 or magic[1] != 0:
            raise ValueError(f"{path}: not an IDX file")
        ndim = magic[3]
        dims = struct.unpack(">" + "I" * ndim, f.read(4 * ndim))
    return {"dtype_code": magic[2], "shape": list(dims)}


def _analyze_tabular(path: str, max_samples: int) -> dict:
    delim = "\t" if path.endswith(".tsv") else ","
    with open(path, newline="") as f:
        rd = csv.reader(f, delimiter=delim)
        header = next(rd, [])
        cols = [{"name": h, "n": 0, "missing": 0, "numeric": 0, "sum": 0.0, "sumsq": 0.0, "min": math.inf, "max": -math.inf,
                 "values": {}} for h in header]
        rows = 0
        for row in rd:
            rows += 1
            if rows > max_samples:
                continue
            for c, v in zip(cols, row):
                c["n"] += 1
                v = v.strip()
                if v == "" or v.lower() in ("na", "nan", "null", "none"):
                    c["missing"] += 1
                    continue
                try:
                    x = float(v)
                    c["numeric"] += 1
                    c["sum"] += x
                    c["sumsq"] += x * x
                    c["min"], c["max"] = min(c["min"], x), max(c["max"], x)
                except ValueError:
                    pass
                if len(c["values"]) <= 64:
                    c["values"][v] = c["values"].get(v, 0) + 1
    out_cols = []
    for c in cols:
        n_ok = c["n"] - c["missing"]
        numeric = n_ok > 0 and c["numeric"] == n_ok
        d = {"name": c["name"], "dtype": "numeric" if numeric else "categorical", "missing": c["missing"],
             "unique": len(c["values"]) if len(c["values"]) <= 64 else None}
        if numeric and c["numeric"]:
            mean = c["sum"] / c["numeric"]
            d.update({"mean": mean, "std": math.sqrt(max(c["sumsq"] / c["numeric"] - mean * mean, 0.0)),
                      "min": c["min"], "max": c["max"]})
        out_cols.append(d)
    target = None
    for cand in ("label", "target", "class", "y"):
        if cand in [h.lower() for h in header]:
            target = header[[h.lower() for h in header].index(cand)]
    if target is None and header:
        target = header[-1]
    tc = next((c for c in cols if c["name"] == target), None)
    classes = dict(tc["values"]) if tc is not None and len(tc["values"]) <= 64 else {}
    task = "classification" if classes and len(classes) <= 50 else "regression"
    return {"num_samples": rows, "num_features": max(len(header) - 1, 0), "columns": out_cols, "target": target,
            "class_counts": classes if task == "classification" else {}, "task": task,
            "missing_values": sum(c["missing"] for c in cols)}


def _analyze_image_folder(path: str, max_samples: int) -> dict:
    classes, total, sizes = {}, 0, {}
    for root, _, files in os.walk(path):
        imgs = [f for f in files if os.path.splitext(f)[1].lower() in IMAGE_EXT]
        if not imgs:
            continue
        rel = os.path.relpath(root, path)
        label = rel.split(os.sep)[-1] if rel != "." else "(root)"
        classes[label] = classes.get(label, 0) + len(imgs)
        total += len(imgs)
        for f in imgs[:max(1, max_samples // max(len(classes), 1))]:
            shp = _image_shape(os.path.join(root, f))
            if shp:
                sizes[shp] = sizes.get(shp, 0) + 1
    common = max(sizes, key=sizes.get) if sizes else None
    return {"num_samples": total, "class_counts": classes, "task": "classification", "num_features": None,
            "image_shape": list(common) if common else None, "distinct_shapes": len(sizes), "missing_values": 0}


def _image_shape(path: str):
    """(channels, height, width) from a PNG / PPM / PGM / BMP header; None for other formats."""
    try:
        with open(path, "rb") as f:
            head = f.read(32)
        if head[:8] == b"\x89PNG\r\n\x1a\n":
            w, h = struct.unpack(">II", head[16:24])
            ch = {0: 1, 2: 3, 3: 3, 4: 2, 6: 4}.get(head[25], 3)
            return (ch, h, w)
        if head[:2] in (b"P5", b"P6"):
            with open(path, "rb") as f:
                toks = f.read(64).split()
            return (3 if head[:2] == b"P6" else 1, int(toks[2]), int(toks[1]))
        if head[:2] == b"BM":
            w, h = struct.unpack("<ii", head[18:26])
            return (3, abs(h), w)
    except (OSError, ValueError, IndexError, struct.error):
        pass
    return None


def _analyze_text(path: str, max_samples: int) -> dict:
    files = [path] if os.path.isfile(path) else [os.path.join(r, f) for r, _, fs in os.walk(path) for f in fs
                                                 if os.path.splitext(f)[1].lower() in TEXT_EXT]
    lines = words = chars = 0
    vocab = set()
    for fp in files:
        with open(fp, errors="replace") as f:
            for line in f:
                lines += 1
                if lines > max_samples:
                    break
                toks = line.split()
                words += len(toks)
                chars += len(line)
                if len(vocab) < 200_000:
                    vocab.update(toks)
    return {"num_samples": lines, "num_files": len(files), "words": words, "characters": chars, "vocabulary": len(vocab),
            "mean_words_per_line": words / max(min(lines, max_samples), 1), "task": "generation", "class_counts": {},
            "num_features": None, "missing_values": 0}


def _analyze_idx(path: str) -> dict:
    files = [path] if os.path.isfile(path) else [os.path.join(path, f) for f in sorted(os.listdir(path)) if "idx" in f.lower()]
    heads = {os.path.basename(f): _idx_header(f) for f in files}
    image_sets = [h for h in heads.values() if len(h["shape"]) >= 3]
    images = max(image_sets, key=lambda h: h["shape"][0]) if image_sets else None
    counts = {}
    label_files = [f for f in files if len(heads[os.path.basename(f)]["shape"]) == 1]
    if label_files:
        import gzip
        lf = max(label_files, key=lambda f: heads[os.path.basename(f)]["shape"][0])
        with (gzip.open if lf.endswith(".gz") else open)(lf, "rb") as f:
            f.read(8)
            for b in f.read(1 << 22):
                counts[str(b)] = counts.get(str(b), 0) + 1
    return {"num_samples": images["shape"][0] if images else None, "files": heads, "task": "classification",
            "image_shape": ([1] + images["shape"][1:] if len(images["shape"]) == 3 else images["shape"][1:]) if images else None,
            "class_counts": counts, "num_features": None, "missing_values": 0}


def analyze_dataset(path: str, dataset_type: str | None = None, max_samples: int = 10_000) -> dict:
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    kind = dataset_type or detect_type(path)
    if kind == "tabular":
        target = path if os.path.isfile(path) else next(os.path.join(r, f) for r, _, fs in os.walk(path) for f in fs
                                                        if os.path.splitext(f)[1].lower() in (".csv", ".tsv"))
        a = _analyze_tabular(target, max_samples)
    elif kind == "image":
        a = _analyze_image_folder(path if os.path.isdir(path) else os.path.dirname(path), max_samples)
    elif kind == "text":
        a = _analyze_text(path, max_samples)
    elif kind == "idx":
        a = _analyze_idx(path)
    else:
        n = sum(len(fs) for _, _, fs in os.walk(path)) if os.path.isdir(path) else 1
        a = {"num_samples": n, "task": "unknown", "class_counts": {}, "num_features": None, "missing_values": 0}
    cc = a.get("class_counts") or {}
    a["num_classes"] = len(cc) or None
    a["imbalance_ratio"] = (max(cc.values()) / max(min(cc.values()), 1)) if cc else None
    a["dataset_type"], a["path"] = kind, os.path.abspath(path)
    a["size_bytes"] = (sum(os.path.getsize(os.path.join(r, f)) for r, _, fs in os.walk(path) for f in fs)
                       if os.path.isdir(path) else os.path.getsize(path))
    a["recommendations"] = recommend_config(a)
    return a


def recommend_config(a: dict) -> dict:
    n = a.get("num_samples") or 0
    kind = a.get("dataset_type")
    batch = 16 if n < 1000 else 32 if n < 10_000 else 64 if n < 100_000 else 128
    rec = {"batch_size": batch, "learning_rate": 1e-3, "optimizer": "adam", "epochs": 20 if n < 10_000 else 10,
           "val_split": 0.2 if n < 5000 else 0.1}
    if kind in ("image", "idx"):
        shp = a.get("image_shape") or [1, 28, 28]
        rec["architecture"] = "lenet" if shp[-1] <= 32 and shp[0] == 1 else "simplecnn" if shp[-1] <= 64 else "resnet18"
        rec["input_size"] = shp
    elif kind == "tabular":
        f = a.get("num_features") or 1
        rec["architecture"], rec["input_size"] = "mlp", [f]
        rec["hidden_sizes"] = [max(32, min(512, 4 * f)), max(16, min(256, 2 * f))]
    elif kind == "text":
        rec.update({"architecture": "gpt2", "learning_rate": 3e-4, "optimizer": "adamw"})
    if a.get("imbalance_ratio") and a["imbalance_ratio"] > 3:
        rec["notes"] = ["classes are imbalanced (ratio %.1f): use a weighted sampler or class weights" % a["imbalance_ratio"]]
    return rec


def preview_dataset(path: str, n: int = 5, dataset_type: str | None = None) -> list:
    kind = dataset_type or detect_type(path)
    if kind == "tabular" and os.path.isfile(path):
        with open(path, newline="") as f:
            rd = csv.DictReader(f, delimiter="\t" if path.endswith(".tsv") else ",")
            return [row for _, row in zip(range(n), rd)]
    if kind == "text":
        fp = path if os.path.isfile(path) else next(os.path.join(r, f) for r, _, fs in os.walk(path) for f in fs)
        with open(fp, errors="replace") as f:
            return [line.rstrip("\n") for _, line in zip(range(n), f)]
    out = []
    for root, _, files in os.walk(path if os.path.isdir(path) else os.path.dirname(path)):
        for f in sorted(files):
            out.append({"file": os.path.relpath(os.path.join(root, f), path), "bytes": os.path.getsize(os.path.join(root, f))})
            if len(out) >= n:
                return out
    return out


def validate_dataset(path: str, num_classes: int | None = None, input_shape: list | None = None,
                     check_missing: bool = True, check_balance: bool = True) -> dict:
    a = analyze_dataset(path)
    issues, warnings = [], []
    if not a.get("num_samples"):
        issues.append("no samples found")
    if num_classes is not None and a.get("num_classes") not in (None, num_classes):
        issues.append(f"expected {num_classes} classes, found {a['num_classes']}")
    if input_shape is not None and a.get("image_shape") and list(input_shape) != list(a["image_shape"]):
        issues.append(f"expected input shape {list(input_shape)}, found {a['image_shape']}")
    if a.get("distinct_shapes", 1) > 1:
        warnings.append(f"{a['distinct_shapes']} distinct image shapes: add a Resize transform")
    if check_missing and a.get("missing_values"):
        warnings.append(f"{a['missing_values']} missing values")
    if check_balance and a.get("imbalance_ratio") and a["imbalance_ratio"] > 3:
        warnings.append(f"class imbalance ratio {a['imbalance_ratio']:.1f}")
    return {"valid": not issues, "issues": issues, "warnings": warnings, "analysis": a}


def generate_config(path: str, fmt: str = "toml") -> str:
    a = analyze_dataset(path)
    r = a["recommendations"]
    cfg = {"project": {"name": os.path.basename(os.path.abspath(path)) or "dataset"},
           "training": {"epochs": r["epochs"], "batch_size": r["batch_size"], "learning_rate": r["learning_rate"],
                        "optimizer": {"name": r["optimizer"]}},
           "model": {"architecture": r.get("architecture", "mlp"), "input_size": r.get("input_size", [1]),
                     "num_classes": a.get("num_classes") or 10},
           "data": {"train_path": a["path"], "format": a["dataset_type"], "val_split": r["val_split"]}}
    if "hidden_sizes" in r:
        cfg["model"]["hidden_sizes"] = r["hidden_sizes"]
    if fmt == "json":
        return json.dumps(cfg, indent=2)
    return _to_toml(cfg)


def _to_toml(d: dict, prefix: str = "") -> str:
    scalars = {k: v for k, v in d.items() if not isinstance(v, dict)}
    tables = {k: v for k, v in d.items() if isinstance(v, dict)}
    out = []
    if prefix and scalars:
        out.append(f"[{prefix}]")
    for k, v in scalars.items():
        out.append(f"{k} = {_toml_value(v)}")
    if scalars:
        out.append("")
    for k, v in tables.items():
        out.append(_to_toml(v, f"{prefix}.{k}" if prefix else k))
    return "\n".join(out)


def _toml_value(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return repr(v)
    if isinstance(v, (list, tuple)):
        return "[" + ", ".join(_toml_value(x) for x in v) + "]"
    return json.dumps(str(v))
