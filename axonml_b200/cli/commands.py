"""Commands that take a model file, in the reference's syntax.

Parity: crates/axonml-cli/src/commands/{eval,predict,report,quant,bench,gpu,hub,inspect,export}.rs
and the argument structs in src/cli.rs (``eval MODEL DATA``, ``predict MODEL INPUT``, ``report MODEL
--data D`` with a confusion matrix / per-class metrics / loss curves in html, json or text, ``quant
convert | info | benchmark | list``, ``bench model | inference | compare | hardware``, ``gpu list |
info | select | bench | memory | status``, ``hub list | info | download | cached | clear``).

The reference rebuilds an MLP from the state dictionary of the file it is given; ``model_from_file``
does the same for every architecture of this package: the configured one when the checkpoint
records it, else the known architecture whose parameter names and shapes match, else a chain of
Linear + ReLU layers read off the 2-D weights."""
from __future__ import annotations

import html
import json
import os
import time

import torch

from .config import ProjectConfig


# ------------------------------------------------------------------------------------------ models
def _state_of(path: str):
    """``(StateDict, checkpoint-or-None)`` of a model file."""
    from ..serialize import load_checkpoint, load_state_dict
    if path.endswith((".axonml", ".bin")):
        try:
            ck = load_checkpoint(path)
            return ck.model_state, ck
        except Exception:  # noqa: BLE001 - a bare state dict in the same container
            pass
    return load_state_dict(path), None


def _known_architectures(tensors: dict):
    from ..vision.models.lenet import LeNet, MLP, SimpleCNN
    yield "lenet", LeNet.new
    for ch, side in ((1, 28), (3, 32)):
        yield "simplecnn", (lambda c=ch, s=side: SimpleCNN(c, _last_out(tensors), s))
    w2 = [(k, v) for k, v in tensors.items() if k.endswith("weight") and v.dim() == 2]
    if w2 and all(k.startswith("layers.") for k in tensors):
        hidden = [int(v.shape[0]) for _, v in w2[:-1]]
        yield "mlp", (lambda: MLP(int(w2[0][1].shape[1]), hidden, int(w2[-1][1].shape[0])))


def _last_out(tensors: dict) -> int:
    w = [v for k, v in tensors.items() if k.endswith("weight") and v.dim() == 2]
    return int(w[-1].shape[0]) if w else 10


def model_from_file(path: str, cfg: ProjectConfig | None = None):
    """``(module in eval mode, architecture name)`` for a checkpoint or state-dict file."""
    from .. import nn
    sd, ck = _state_of(path)
    tensors = sd.to_tensors()
    shapes = {k: tuple(v.shape) for k, v in tensors.items()}
    if cfg is None and ck is not None and ck.config.get("architecture"):
        cfg = ProjectConfig()
        cfg.model.architecture = str(ck.config["architecture"])
    if cfg is not None:
        from .main import build_model
        first = next((v for k, v in tensors.items() if k.endswith("weight") and v.dim() == 2), None)
        if cfg.model.architecture.lower() == "mlp" and first is not None:
            w2 = [v for k, v in tensors.items() if k.endswith("weight") and v.dim() == 2]
            cfg.model.input_size, cfg.model.hidden_sizes = [int(first.shape[1])], [int(v.shape[0]) for v in w2[:-1]]
            cfg.model.num_classes = int(w2[-1].shape[0])
        try:
            m = build_model(cfg)
            if {k: tuple(p.shape) for k, p in m.named_parameters()} == {k: s for k, s in shapes.items() if k in dict(m.named_parameters())}:
                sd.load_into(m, strict=False)
                return m.eval(), cfg.model.architecture.lower()
        except (SystemExit, RuntimeError, ValueError):
            pass
    for name, make in _known_architectures(tensors):
        try:
            m = make()
        except Exception:  # noqa: BLE001 - the candidate does not fit these tensors
            continue
        own = {k: tuple(p.shape) for k, p in m.named_parameters()}
        if own == {k: shapes[k] for k in own if k in shapes} and set(own) <= set(shapes):
            sd.load_into(m, strict=False)
            return m.eval(), name
    # generic: 2-D weights in file order are Linear layers with ReLU between them
    layers = nn.Sequential()
    w2 = [(k, v) for k, v in tensors.items() if k.endswith("weight") and v.dim() == 2]
    if not w2:
        raise SystemExit(f"{path}: cannot rebuild a model from these tensors (no 2-D weights and no recorded architecture)")
    for i, (k, w) in enumerate(w2):
        b = tensors.get(k[:-len("weight")] + "bias")
        lin = nn.Linear(int(w.shape[1]), int(w.shape[0]), bias=b is not None)
        with torch.no_grad():
            lin.weight.copy_(w.float())
            if b is not None:
                lin.bias.copy_(b.float())
        layers.add(lin)
        if i + 1 < len(w2):
            layers.add(nn.ReLU())
    return layers.eval(), "sequential-mlp"


def _input_width(model) -> int | None:
    for p in model.parameters():
        if p.dim() == 2:
            return int(p.shape[1])
        if p.dim() == 4:
            return None
    return None


def _feed(model, x: torch.Tensor) -> torch.Tensor:
    """Runs ``model`` on a batch, flattening images when the model starts with a Linear layer."""
    w = _input_width(model)
    if w is not None and x.dim() > 2:
        x = x.flatten(1)
    return model(x)


# -------------------------------------------------------------------------------------------- data
def detect_data_format(path: str) -> str | None:
    if not os.path.exists(path):
        return None
    names = set(os.listdir(path)) if os.path.isdir(path) else {os.path.basename(path)}
    if any("idx3-ubyte" in n for n in names):
        return "mnist"
    if any(n.startswith("data_batch_") or n == "test_batch.bin" for n in names):
        return "cifar10"
    if {"train.bin", "test.bin"} & names:
        return "cifar100"
    if any(n.endswith((".csv", ".tsv")) for n in names):
        return "csv"
    return None


def dataset_from_path(path: str, fmt: str | None = None, train: bool = False):
    """Dataset for a path (or a built-in synthetic set named by ``path``)."""
    from ..data.dataset import TensorDataset
    from ..vision import datasets as D
    key = (fmt or "").lower() or path.lower()
    if key in ("synthetic", "synthetic-mnist"):
        return D.SyntheticMNIST(512)
    if key == "synthetic-cifar":
        return D.SyntheticCIFAR(512)
    fmt = (fmt or detect_data_format(path) or "").lower()
    if fmt in ("mnist", "fashion-mnist", "fashionmnist"):
        cls = D.MNIST if fmt == "mnist" else D.FashionMNIST
        try:
            return cls(path, train=train)
        except FileNotFoundError:
            return cls(path, train=not train)
    if fmt == "cifar10":
        return D.CIFAR10(path, train=train)
    if fmt == "cifar100":
        return D.CIFAR100(path, train=train)
    if fmt in ("csv", "tsv"):
        import csv
        f = path if os.path.isfile(path) else next(os.path.join(path, n) for n in sorted(os.listdir(path)) if n.endswith((".csv", ".tsv")))
        with open(f, newline="") as fh:
            rows = list(csv.reader(fh, delimiter="\t" if f.endswith(".tsv") else ","))
        head, body = rows[0], rows[1:]
        try:
            [float(v) for v in head]
            body = rows
        except ValueError:
            pass
        labels = sorted({r[-1] for r in body})
        lut = {l: i for i, l in enumerate(labels)}
        x = torch.tensor([[float(v) for v in r[:-1]] for r in body], dtype=torch.float32)
        y = torch.tensor([lut[r[-1]] for r in body], dtype=torch.long)
        ds = TensorDataset(x, y)
        ds.class_names_ = labels
        return ds
    raise SystemExit(f"cannot tell the format of {path!r}: pass --format mnist | fashion-mnist | cifar10 | cifar100 | csv | synthetic")


# ---------------------------------------------------------------------------------------- metrics
def classification_metrics(confusion: torch.Tensor, class_names=None, loss: float | None = None) -> dict:
    """Accuracy, per-class precision / recall / F1 / support and their macro and weighted averages
    from a confusion matrix ``[true, predicted]`` (report.rs:475-595)."""
    c = confusion.double()
    n = c.shape[0]
    total = float(c.sum())
    per_class = []
    for i in range(n):
        tp = float(c[i, i])
        fp, fn = float(c[:, i].sum()) - tp, float(c[i].sum()) - tp
        prec = tp / (tp + fp) if tp + fp > 0 else 0.0
        rec = tp / (tp + fn) if tp + fn > 0 else 0.0
        f1 = 2 * prec * rec / (prec + rec) if prec + rec > 0 else 0.0
        per_class.append({"class_id": i, "class_name": (class_names[i] if class_names and i < len(class_names) else str(i)),
                          "precision": prec, "recall": rec, "f1_score": f1, "support": int(c[i].sum())})
    valid = [p for p in per_class if p["support"] > 0]
    mp = sum(p["precision"] for p in valid) / len(valid) if valid else 0.0
    mr = sum(p["recall"] for p in valid) / len(valid) if valid else 0.0
    return {"accuracy": float(c.diag().sum()) / total if total else 0.0, "total_samples": int(total), "loss": loss,
            "macro_precision": mp, "macro_recall": mr, "macro_f1": 2 * mp * mr / (mp + mr) if mp + mr > 0 else 0.0,
            "weighted_f1": sum(p["f1_score"] * p["support"] for p in per_class) / total if total else 0.0,
            "per_class": per_class, "confusion_matrix": confusion.long().tolist()}


@torch.no_grad()
def evaluate(model, dataset, batch_size: int = 32, device="cpu", num_classes: int | None = None) -> tuple:
    """``(confusion matrix, mean cross-entropy)`` of ``model`` over ``dataset``."""
    from ..data import DataLoader
    dev = torch.device(device)
    model = model.to(dev).eval()
    conf, loss_sum, count = None, 0.0, 0
    for b in DataLoader(dataset, batch_size):
        x, y = b.data.to(dev), b.targets.to(dev).long()
        if y.dim() > 1:
            y = y.argmax(-1)
        logits = _feed(model, x).float()
        k = num_classes or logits.shape[-1]
        if conf is None:
            conf = torch.zeros(k, k, dtype=torch.long)
        pred = logits.argmax(-1)
        conf += torch.bincount((y.clamp(max=k - 1) * k + pred.clamp(max=k - 1)).cpu(), minlength=k * k).view(k, k)
        loss_sum += float(torch.nn.functional.cross_entropy(logits, y.clamp(max=logits.shape[-1] - 1), reduction="sum"))
        count += y.numel()
    if conf is None:
        raise SystemExit("the dataset is empty")
    return conf, loss_sum / max(count, 1)


def load_history(path: str | None) -> list:
    """Per-epoch records from a training log (JSON lines or a JSON list / dict of lists)."""
    if not path or not os.path.exists(path):
        return []
    from ..tui.views.training import parse_training_log
    try:
        s = parse_training_log(path)
    except (OSError, ValueError):
        return []
    return [{"epoch": m.epoch, "train_loss": m.train_loss, "val_loss": m.val_loss, "train_acc": m.train_acc, "val_acc": m.val_acc}
            for m in s.metrics_history]


def _svg_curve(points, w=520, h=160, colour="#14b8a6") -> str:
    if len(points) < 2:
        return ""
    xs, ys = [p[0] for p in points], [p[1] for p in points]
    x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
    sx = lambda x: 10 + (x - x0) / ((x1 - x0) or 1) * (w - 20)
    sy = lambda y: h - 10 - (y - y0) / ((y1 - y0) or 1) * (h - 20)
    pts = " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in points)
    return f'<polyline fill="none" stroke="{colour}" stroke-width="2" points="{pts}"/>'


def render_report(metrics: dict, model_name: str, fmt: str, history=None, confusion: bool = True, per_class: bool = True,
                  curves: bool = True) -> str:
    history = history or []
    if fmt == "json":
        out = dict(metrics)
        if not confusion:
            out.pop("confusion_matrix", None)
        if not per_class:
            out.pop("per_class", None)
        return json.dumps({"model": model_name, "metrics": out, "history": history if curves else []}, indent=1)
    head = [("Accuracy", metrics["accuracy"]), ("Macro precision", metrics["macro_precision"]), ("Macro recall", metrics["macro_recall"]),
            ("Macro F1", metrics["macro_f1"]), ("Weighted F1", metrics["weighted_f1"])]
    if fmt == "text":
        lines = [f"Evaluation report: {model_name}", f"Samples: {metrics['total_samples']}"]
        lines += [f"{k:18s} {v:.4f}" for k, v in head]
        if metrics.get("loss") is not None:
            lines.append(f"{'Loss':18s} {metrics['loss']:.4f}")
        if per_class:
            lines += ["", f"{'class':16s} {'precision':>9s} {'recall':>9s} {'f1':>9s} {'support':>8s}"]
            lines += [f"{p['class_name'][:16]:16s} {p['precision']:9.4f} {p['recall']:9.4f} {p['f1_score']:9.4f} {p['support']:8d}"
                      for p in metrics["per_class"]]
        if confusion:
            lines += ["", "Confusion matrix (rows: true class, columns: predicted)"]
            lines += [" ".join(f"{v:6d}" for v in row) for row in metrics["confusion_matrix"]]
        if curves and history:
            lines += ["", "epoch  train_loss  val_loss"]
            lines += [f"{r['epoch']:5d}  {r['train_loss']:10.4f}  {'' if r['val_loss'] is None else format(r['val_loss'], '.4f')}" for r in history]
        return "\n".join(lines)
    e = html.escape
    parts = [f"<html><head><meta charset='utf-8'><title>{e(model_name)}</title><style>body{{font-family:sans-serif;margin:2em}}"
             "table{border-collapse:collapse}td,th{border:1px solid #ccc;padding:4px 8px;text-align:right}th{background:#f5ebe0}</style></head><body>",
             f"<h1>Evaluation report: {e(model_name)}</h1><p>{metrics['total_samples']} samples</p><table>"]
    parts += [f"<tr><th>{k}</th><td>{v:.4f}</td></tr>" for k, v in head]
    if metrics.get("loss") is not None:
        parts.append(f"<tr><th>Loss</th><td>{metrics['loss']:.4f}</td></tr>")
    parts.append("</table>")
    if per_class:
        parts.append("<h2>Per-class metrics</h2><table><tr><th>class</th><th>precision</th><th>recall</th><th>F1</th><th>support</th></tr>")
        parts += [f"<tr><td>{e(p['class_name'])}</td><td>{p['precision']:.4f}</td><td>{p['recall']:.4f}</td><td>{p['f1_score']:.4f}</td>"
                  f"<td>{p['support']}</td></tr>" for p in metrics["per_class"]]
        parts.append("</table>")
    if confusion:
        cm = metrics["confusion_matrix"]
        top = max((max(r) for r in cm), default=1) or 1
        parts.append("<h2>Confusion matrix</h2><table><tr><th>true \\ predicted</th>" + "".join(f"<th>{i}</th>" for i in range(len(cm))) + "</tr>")
        for i, row in enumerate(cm):
            cells = "".join(f"<td style='background:rgba(20,184,166,{v / top:.2f})'>{v}</td>" for v in row)
            parts.append(f"<tr><th>{i}</th>{cells}</tr>")
        parts.append("</table>")
    if curves and history:
        tr = [(r["epoch"], r["train_loss"]) for r in history]
        va = [(r["epoch"], r["val_loss"]) for r in history if r["val_loss"] is not None]
        parts.append("<h2>Loss curves</h2><svg width='520' height='160' style='border:1px solid #ccc'>" + _svg_curve(tr) + _svg_curve(va, colour="#c4a484")
                     + "</svg><p>teal: training, tan: validation</p>")
    parts.append("</body></html>")
    return "".join(parts)


# ------------------------------------------------------------------------------------------ input
def load_input(spec: str) -> torch.Tensor:
    """Input of ``predict``: a .json / .csv / .npy / .pt file, a JSON array (optionally wrapped as
    ``{"data": ...}`` or ``{"input": ...}``) or comma-separated numbers (predict.rs:176-290)."""
    def from_json(text):
        j = json.loads(text)
        if isinstance(j, dict):
            j = j.get("data", j.get("input", j.get("inputs", j.get("features"))))
            if j is None:
                raise SystemExit('JSON input needs a "data" (or "input") array')
        return torch.tensor(j, dtype=torch.float32)

    if os.path.isfile(spec):
        if spec.endswith(".npy"):
            import numpy as np
            return torch.from_numpy(np.load(spec)).float()
        if spec.endswith((".pt", ".pth")):
            return torch.as_tensor(torch.load(spec, weights_only=True)).float()
        with open(spec) as f:
            text = f.read().strip()
        if spec.endswith(".json") or text[:1] in "[{":
            return from_json(text)
        rows = [[float(v) for v in line.replace(";", ",").split(",") if v.strip()] for line in text.splitlines() if line.strip()]
        return torch.tensor(rows if len(rows) > 1 else rows[0], dtype=torch.float32)
    s = spec.strip()
    if s[:1] in "[{":
        return from_json(s)
    if "," in s:
        return torch.tensor([float(v) for v in s.split(",") if v.strip()], dtype=torch.float32)
    raise SystemExit(f"Cannot parse input: {spec}. Expected file path, JSON, or comma-separated values.")


def shape_input_for(model, x: torch.Tensor) -> torch.Tensor:
    """Adds the batch dimension (and image dimensions for convolutional models) a flat input lacks."""
    w = _input_width(model)
    if w is not None:
        return x.reshape(-1, w) if x.numel() % w == 0 else x.reshape(1, -1)
    first = next(p for p in model.parameters() if p.dim() == 4)
    c = int(first.shape[1])
    if x.dim() == 4:
        return x
    if x.dim() == 3:
        return x.unsqueeze(0)
    side = int(round((x.numel() / c) ** 0.5))
    return x.reshape(-1, c, side, side)


# ------------------------------------------------------------------------------------------- quant
QUANT_TYPES = [("q8_0", "8-bit blocks of 32, fp16 scale", 8.5), ("q4_0", "4-bit blocks of 32, fp16 scale", 4.5),
               ("q4_1", "4-bit blocks of 32, fp16 scale + minimum", 5.0), ("q5_0", "5-bit blocks of 32, fp16 scale", 5.5),
               ("q5_1", "5-bit blocks of 32, fp16 scale + minimum", 6.0), ("q4_k", "4-bit super-blocks of 256 with 6-bit sub-scales", 4.5),
               ("f16", "half precision", 16.0), ("f32", "single precision", 32.0)]


def quant_type(name: str):
    from ..quant.types import QuantType
    qt = QuantType.from_str(name.lower()) if hasattr(QuantType, "from_str") else None
    if qt is None:
        try:
            qt = QuantType[name.upper()]
        except KeyError:
            raise SystemExit(f"unknown quantisation type {name!r}; try: " + ", ".join(n for n, _, _ in QUANT_TYPES)) from None
    return qt


def quant_info(path: str, detailed: bool = False) -> dict:
    """Tensors of a model file by storage type, with the bytes they take."""
    from ..server.app.registry import detect_format
    rows = []
    if detect_format(path) == "gguf":
        from ..quant.gguf import read_gguf
        g = read_gguf(path)
        for name in g.tensor_names():
            info = g.tensor_info(name)
            rows.append({"name": name, "shape": info["shape"], "type": info["type"], "numel": info["numel"]})
    else:
        sd, _ = _state_of(path)
        for k, v in sd.to_tensors().items():
            rows.append({"name": k, "shape": list(v.shape), "type": str(v.dtype).replace("torch.", ""), "numel": v.numel()})
    by_type: dict = {}
    for r in rows:
        t = by_type.setdefault(r["type"], {"tensors": 0, "parameters": 0})
        t["tensors"] += 1
        t["parameters"] += r["numel"]
    out = {"path": path, "file_bytes": os.path.getsize(path), "tensors": len(rows), "parameters": sum(r["numel"] for r in rows), "by_type": by_type}
    out["bits_per_parameter"] = 8.0 * out["file_bytes"] / max(out["parameters"], 1)
    if detailed:
        out["entries"] = rows
    return out


def quant_benchmark(path: str, types, iterations: int = 10, min_numel: int = 1024) -> list:
    """Per type: compressed size, round-trip error and quantise / dequantise time over the file's weight matrices."""
    from ..quant.quantize import compute_quantization_error, dequantize_tensor, quantize_tensor
    sd, _ = _state_of(path)
    mats = [v.float() for v in sd.to_tensors().values() if v.dim() >= 2 and v.numel() >= min_numel]
    rows = []
    for name in types:
        qt = quant_type(name)
        use = [m for m in mats if m.shape[-1] % qt.block_size() == 0]
        if not use:
            rows.append({"type": name, "tensors": 0})
            continue
        t0 = time.perf_counter()
        for _ in range(iterations):
            qs = [quantize_tensor(m, qt) for m in use]
        tq = (time.perf_counter() - t0) / iterations
        t0 = time.perf_counter()
        for _ in range(iterations):
            ds = [dequantize_tensor(q) for q in qs]
        td = (time.perf_counter() - t0) / iterations
        orig = sum(m.numel() * 4 for m in use)
        comp = sum(q.size_bytes() for q in qs)
        err = sum(compute_quantization_error(m, d.view_as(m)) for m, d in zip(use, ds)) / len(use)
        rows.append({"type": name, "tensors": len(use), "original_bytes": orig, "quantized_bytes": comp, "compression_ratio": orig / comp,
                     "mean_rmse": err, "quantize_ms": tq * 1e3, "dequantize_ms": td * 1e3})
    return rows


# ------------------------------------------------------------------------------------------- bench
def _time_model(model, x, iterations: int, warmup: int) -> dict:
    with torch.no_grad():
        for _ in range(warmup):
            _feed(model, x)
        if x.is_cuda:
            torch.cuda.synchronize()
        times = []
        for _ in range(iterations):
            if x.is_cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                _feed(model, x)
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            else:
                t0 = time.perf_counter()
                _feed(model, x)
                times.append((time.perf_counter() - t0) * 1e3)
    times.sort()
    pick = lambda q: times[min(int(q * len(times)), len(times) - 1)]
    mean = sum(times) / len(times)
    return {"iterations": iterations, "mean_ms": mean, "min_ms": times[0], "max_ms": times[-1], "p50_ms": pick(0.5), "p95_ms": pick(0.95),
            "p99_ms": pick(0.99), "throughput_per_s": x.shape[0] / (mean / 1e3) if mean else 0.0}


def example_input(model, batch: int, device) -> torch.Tensor:
    w = _input_width(model)
    if w is not None:
        return torch.randn(batch, w, device=device)
    first = next(p for p in model.parameters() if p.dim() == 4)
    side = 32 if int(first.shape[1]) == 3 else 28
    return torch.randn(batch, int(first.shape[1]), side, side, device=device)


def bench_model_file(path: str, iterations: int, warmup: int, batch_size: int, device: str) -> dict:
    model, arch = model_from_file(path)
    dev = torch.device("cuda" if device == "auto" and torch.cuda.is_available() else ("cpu" if device == "auto" else device))
    model = model.to(dev)
    r = _time_model(model, example_input(model, batch_size, dev), iterations, warmup)
    return {"model": os.path.basename(path), "architecture": arch, "device": str(dev), "batch_size": batch_size,
            "parameters": sum(p.numel() for p in model.parameters()), **r}


# --------------------------------------------------------------------------------------------- gpu
def gpu_devices() -> list:
    out = []
    for i in range(torch.cuda.device_count() if torch.cuda.is_available() else 0):
        p = torch.cuda.get_device_properties(i)
        free, total = torch.cuda.mem_get_info(i)
        out.append({"index": i, "name": p.name, "backend": "cuda", "compute_capability": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                    "memory_total_bytes": total, "memory_free_bytes": free})
    return out


def gpu_selection_file() -> str:
    base = os.environ.get("AXONML_CONFIG_DIR") or os.path.join(os.path.expanduser("~"), ".config", "axonml")
    return os.path.join(base, "gpu.json")


def gpu_selected():
    try:
        with open(gpu_selection_file()) as f:
            return json.load(f).get("device")
    except (OSError, ValueError):
        return None


def gpu_select(device: str, persistent: bool) -> dict:
    """Checks that ``device`` (an index, ``cuda:N`` or ``cpu``) exists; with ``persistent`` it is
    written to the user's configuration, where ``train --device auto`` picks it up."""
    name = device if not device.isdigit() else f"cuda:{device}"
    if name != "cpu":
        idx = int(name.split(":")[1]) if ":" in name else 0
        if idx >= (torch.cuda.device_count() if torch.cuda.is_available() else 0):
            raise SystemExit(f"no such GPU: {device} ({torch.cuda.device_count() if torch.cuda.is_available() else 0} CUDA devices present)")
    if persistent:
        os.makedirs(os.path.dirname(gpu_selection_file()), exist_ok=True)
        with open(gpu_selection_file(), "w") as f:
            json.dump({"device": name}, f)
    return {"selected": name, "persistent": persistent}


def gpu_bench(index: int, iterations: int) -> dict:
    dev = torch.device("cuda", index)
    n = 4096
    a = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
    b = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
    from ..ops.gemm import gemm_bf16, gemm_supported
    f = (lambda: gemm_bf16(a, b)) if gemm_supported(a, b) else (lambda: a @ b.t())
    for _ in range(3):
        f()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iterations):
        f()
    e1.record()
    torch.cuda.synchronize(dev)
    gemm = 2 * n ** 3 * iterations / (e0.elapsed_time(e1) / 1e3) / 1e12
    src = torch.empty(1 << 28, dtype=torch.uint8, device=dev)
    dst = torch.empty_like(src)
    dst.copy_(src)
    e0.record()
    for _ in range(iterations):
        dst.copy_(src)
    e1.record()
    torch.cuda.synchronize(dev)
    return {"device": index, "bf16_gemm_tflops": gemm, "copy_gbs": 2 * src.numel() * iterations / (e0.elapsed_time(e1) / 1e3) / 1e9}
