"""Workspace commands of the CLI: ``upload``, ``data``, ``scaffold``, ``zip``, ``rename``, ``load``
and ``analyze``.

Parity: crates/axonml-cli/src/commands/{upload,data,scaffold,zip,rename,load,analyze}.rs and their
argument structs (cli.rs:568-1215).  The workspace is a JSON file (``.axonml/workspace.json`` in
the current directory) naming the loaded model and dataset; model files live under ``./models``,
datasets under ``./datasets``.  ``scaffold`` writes a Python training project for this package
where the reference writes a Rust one."""
from __future__ import annotations

import json
import os
import shutil
import time
import zipfile

WORKSPACE = os.path.join(".axonml", "workspace.json")


# ----------------------------------------------------------------------------- helpers
def _ws_load() -> dict:
    try:
        with open(WORKSPACE) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {"model": None, "dataset": None}


def _ws_save(ws: dict) -> None:
    os.makedirs(os.path.dirname(WORKSPACE), exist_ok=True)
    with open(WORKSPACE, "w") as f:
        json.dump(ws, f, indent=1)


def model_summary(path: str) -> dict:
    """Format, tensor count, parameter count, bytes and per-layer rows of a model file."""
    from ..server.app.registry import detect_format
    fmt = detect_format(path)
    rows = []
    if fmt == "gguf":
        from ..quant.gguf import read_gguf
        g = read_gguf(path)
        for name in g.tensor_names():
            info = g.tensor_info(name)
            rows.append({"name": name, "shape": info["shape"], "dtype": info["type"], "numel": info["numel"]})
    elif fmt == "onnx":
        from ..onnx import load_onnx
        m = load_onnx(path)
        for name, t in getattr(m, "initializers", {}).items():
            rows.append({"name": name, "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "numel": t.numel()})
    else:
        from ..serialize import load_checkpoint, load_state_dict
        try:
            sd = load_checkpoint(path).model_state
        except Exception:  # noqa: BLE001 - not a checkpoint container: a bare state dict
            sd = load_state_dict(path)
        for k, v in sd.to_tensors().items():
            rows.append({"name": k, "shape": list(v.shape), "dtype": str(v.dtype).replace("torch.", ""), "numel": v.numel()})
    layers = {}
    for r in rows:
        stem = r["name"].rsplit(".", 1)[0] if "." in r["name"] else r["name"]
        layers.setdefault(stem, 0)
        layers[stem] += r["numel"]
    return {"path": os.path.abspath(path), "format": fmt, "file_bytes": os.path.getsize(path), "tensors": len(rows),
            "parameters": sum(r["numel"] for r in rows), "layers": [{"name": k, "parameters": v} for k, v in layers.items()],
            "entries": rows}


def _print_model(s: dict, detailed: bool) -> None:
    print(f"{s['path']}\n  format {s['format']}  {s['file_bytes']:,} bytes  {s['tensors']} tensors  {s['parameters']:,} parameters")
    if detailed:
        for r in s["entries"]:
            print(f"  {r['name']:56s} {str(r['shape']):22s} {r['dtype']}")
    else:
        for l in s["layers"][:40]:
            print(f"  {l['name']:56s} {l['parameters']:>12,}")


def _emit(obj, fmt: str, output: str | None) -> None:
    text = json.dumps(obj, indent=2, default=str) if fmt == "json" else _as_text(obj)
    if output:
        with open(output, "w") as f:
            f.write(text + "\n")
        print(f"wrote {output}")
    else:
        print(text)


def _as_text(obj, indent: int = 0) -> str:
    pad = "  " * indent
    if isinstance(obj, dict):
        out = []
        for k, v in obj.items():
            if isinstance(v, (dict, list)) and v:
                out.append(f"{pad}{k}:")
                out.append(_as_text(v, indent + 1))
            else:
                out.append(f"{pad}{k}: {v}")
        return "\n".join(out)
    if isinstance(obj, list):
        return "\n".join(_as_text(v, indent) if isinstance(v, (dict, list)) else f"{pad}- {v}" for v in obj[:50])
    return pad + str(obj)


# ----------------------------------------------------------------------------- upload
def cmd_upload(a) -> None:
    if not os.path.isfile(a.path):
        raise SystemExit(f"no such file: {a.path}")
    name = a.name or os.path.splitext(os.path.basename(a.path))[0]
    ext = os.path.splitext(a.path)[1]
    dest_dir = a.dest or "models"
    os.makedirs(dest_dir, exist_ok=True)
    dest = os.path.join(dest_dir, f"{name}{('-' + a.version) if a.version else ''}{ext}")
    if os.path.exists(dest) and not a.overwrite:
        raise SystemExit(f"{dest} exists (use --overwrite)")
    summary = model_summary(a.path) if (a.validate or a.info) else None      # unreadable files fail before the copy
    shutil.copy2(a.path, dest)
    meta = {"name": name, "description": a.description or "", "version": a.version, "source": os.path.abspath(a.path),
            "uploaded_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    if summary:
        meta.update({k: summary[k] for k in ("format", "tensors", "parameters", "file_bytes")})
    with open(dest + ".meta.json", "w") as f:
        json.dump(meta, f, indent=1)
    print(f"uploaded {name} -> {dest}")
    if summary and a.info:
        _print_model(summary, False)


# ----------------------------------------------------------------------------- data
def cmd_data(a) -> None:
    from ..data import analysis as A
    act = a.action
    if act == "upload":
        name = a.name or os.path.basename(os.path.normpath(a.path))
        dest = os.path.join(a.dest or "datasets", name)
        if os.path.exists(dest):
            raise SystemExit(f"{dest} exists")
        os.makedirs(os.path.dirname(dest) or ".", exist_ok=True)
        (shutil.copytree if os.path.isdir(a.path) else shutil.copy2)(a.path, dest)
        meta = {"name": name, "type": a.type or A.detect_type(dest), "task": a.task, "split": a.split}
        with open((dest if os.path.isdir(dest) else dest + ".d") + ".meta.json", "w") as f:
            json.dump(meta, f, indent=1)
        print(f"uploaded dataset {name} -> {dest} ({meta['type']})")
        if a.analyze:
            _emit(A.analyze_dataset(dest, a.type), "text", None)
    elif act == "analyze":
        res = A.analyze_dataset(a.path, a.type, a.max_samples)
        if not a.detailed:
            res.pop("columns", None)
        if not a.recommend:
            res.pop("recommendations", None)
        _emit(res, a.format, a.output)
    elif act == "list":
        root = a.path or "datasets"
        for d in sorted(os.listdir(root)) if os.path.isdir(root) else []:
            p = os.path.join(root, d)
            if d.endswith(".meta.json"):
                continue
            line = f"{d:32s} {A.detect_type(p):10s}"
            if a.detailed:
                an = A.analyze_dataset(p)
                line += f" samples={an.get('num_samples')} classes={an.get('num_classes')} bytes={an.get('size_bytes'):,}"
            print(line)
    elif act == "config":
        text = A.generate_config(a.path, a.format if a.format in ("toml", "json") else "toml")
        if a.output:
            with open(a.output, "w") as f:
                f.write(text)
            print(f"wrote {a.output}")
        else:
            print(text)
    elif act == "preview":
        rows = A.preview_dataset(a.path, a.num_samples)
        if a.random:
            import random
            random.shuffle(rows)
        for r in rows:
            print(r)
    elif act == "validate":
        shape = [int(x) for x in a.input_shape.split(",")] if a.input_shape else None
        res = A.validate_dataset(a.path, a.num_classes, shape, a.check_missing, a.check_balance)
        print("valid" if res["valid"] else "INVALID")
        for i in res["issues"]:
            print("  issue:  ", i)
        for w in res["warnings"]:
            print("  warning:", w)
        if not res["valid"]:
            raise SystemExit(1)


# ----------------------------------------------------------------------------- scaffold
TEMPLATES = {
    "training": "a training script with a TOML configuration, checkpoints and validation accuracy",
    "evaluation": "an evaluation script that loads a checkpoint and reports accuracy and a confusion matrix",
    "inference": "a prediction script plus an HTTP inference server entry point",
    "full": "training + evaluation + inference",
}

_TRAIN_PY = '''"""Training entry point generated by `axonml scaffold`."""
import torch
from axonml_b200 import nn, optim
from axonml_b200.cli.config import ProjectConfig
from axonml_b200.cli.main import build_datasets, build_model
from axonml_b200.data import DataLoader
from axonml_b200.serialize import save_state_dict
from axonml_b200.serialize.state_dict import StateDict
{wandb_import}

def main():
    cfg = ProjectConfig.load("axonml.toml")
    torch.manual_seed(cfg.training.seed)
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = build_model(cfg).to(device)
    train_ds, val_ds = build_datasets(cfg)
    loader = DataLoader(train_ds, cfg.training.batch_size, shuffle=True)
    opt = optim.AdamW(list(model.parameters()), cfg.training.learning_rate)
    loss_fn = nn.{loss}()
{wandb_init}
    for epoch in range(cfg.training.epochs):
        total, n = 0.0, 0
        for batch in loader:
            x, y = batch.data.to(device), batch.targets.to(device)
{augment}
            opt.zero_grad()
            loss = loss_fn(model(x), y)
            loss.backward()
            opt.step()
            total, n = total + float(loss.detach()), n + 1
        print(f"epoch {{epoch + 1}}: loss {{total / max(n, 1):.4f}}")
{wandb_log}
    save_state_dict(StateDict.from_module(model), "output/model.axonml")
{wandb_finish}

if __name__ == "__main__":
    main()
'''

_EVAL_PY = '''"""Evaluation entry point generated by `axonml scaffold`."""
import sys
import torch
from axonml_b200.cli.config import ProjectConfig
from axonml_b200.cli.main import build_datasets, build_model
from axonml_b200.data import DataLoader
from axonml_b200.serialize import load_state_dict


def main(path="output/model.axonml"):
    cfg = ProjectConfig.load("axonml.toml")
    model = build_model(cfg).eval()
    load_state_dict(path).load_into(model, strict=False)
    _, val_ds = build_datasets(cfg)
    k = cfg.model.num_classes
    conf = torch.zeros(k, k, dtype=torch.long)
    with torch.no_grad():
        for b in DataLoader(val_ds, cfg.training.batch_size):
            pred = model(b.data).argmax(-1)
            for t, p in zip(b.targets.tolist(), pred.tolist()):
                conf[t, p] += 1
    print(f"accuracy {{conf.diag().sum().item() / max(conf.sum().item(), 1):.4f}}")
    print(conf)


if __name__ == "__main__":
    main(*sys.argv[1:])
'''

_INFER_PY = '''"""Inference entry point generated by `axonml scaffold`: `python infer.py serve` or `python infer.py <v1> <v2> ...`."""
import sys
from axonml_b200.server import AxonmlHTTPServer, InferenceServer


def main():
    srv = InferenceServer()
    srv.load("default", "output/model.axonml")
    if sys.argv[1:] == ["serve"]:
        AxonmlHTTPServer("127.0.0.1", 3021, srv).serve_forever()
    else:
        print(srv.predict("default", [float(v) for v in sys.argv[1:]]))


if __name__ == "__main__":
    main()
'''


def cmd_scaffold(a) -> None:
    if a.action == "templates":
        for k, v in TEMPLATES.items():
            print(f"{k:12s} {v}" if a.detailed else k)
        return
    if a.template not in TEMPLATES:
        raise SystemExit(f"unknown template {a.template!r}; choose from {', '.join(TEMPLATES)}")
    root = os.path.join(a.output or ".", a.name)
    if os.path.exists(root):
        if not a.overwrite:
            raise SystemExit(f"{root} exists (use --overwrite)")
        shutil.rmtree(root)
    os.makedirs(os.path.join(root, "output"))
    from .config import ProjectConfig
    cfg = ProjectConfig()
    cfg.project.name = a.name
    cfg.model.architecture = a.arch
    if getattr(a, "model", None):
        cfg.model.path = a.model
    if getattr(a, "data", None):
        cfg.data.train_path = a.data
    cfg.data.format = "synthetic-mnist"
    with open(os.path.join(root, "axonml.toml"), "w") as f:
        f.write(cfg.to_toml())
    files = []
    if a.template in ("training", "full"):
        wb = a.wandb
        src = _TRAIN_PY.format(
            loss="MSELoss" if a.task == "regression" else "CrossEntropyLoss",
            wandb_import="from axonml_b200.integrations import WandbRun" if wb else "",
            wandb_init='    run = WandbRun(cfg.project.name, config={"lr": cfg.training.learning_rate})' if wb else "",
            wandb_log='        run.log({"loss": total / max(n, 1), "epoch": epoch + 1})' if wb else "",
            wandb_finish="    run.finish()" if wb else "",
            augment="            x = x + 0.01 * torch.randn_like(x)          # noise augmentation" if a.augment else "")
        files.append(("train.py", src))
    if a.template in ("evaluation", "full"):
        files.append(("evaluate.py", _EVAL_PY.replace("{{", "{").replace("}}", "}")))
    if a.template in ("inference", "full"):
        files.append(("infer.py", _INFER_PY))
    files.append(("README.md", f"# {a.name}\n\nGenerated by `axonml scaffold generate` ({a.template} template, {a.task}, "
                                f"{a.arch}).\n\n    python train.py\n"))
    for fn, src in files:
        with open(os.path.join(root, fn), "w") as f:
            f.write(src)
    print(f"created {root}: " + ", ".join(fn for fn, _ in files) + ", axonml.toml")


# ----------------------------------------------------------------------------- zip bundles
def cmd_zip(a) -> None:
    if a.action == "create":
        a.output = getattr(a, "output_opt", None) or a.output
        if not a.output:
            raise SystemExit("zip create needs an output file (-o bundle.zip)")
        if os.path.exists(a.output) and not a.overwrite:
            raise SystemExit(f"{a.output} exists (use --overwrite)")
        if not (a.model or a.data):
            raise SystemExit("give --model and/or --data")
        manifest = {"format": "axonml-bundle-v1", "created_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
                    "model": None, "dataset": None, "config": []}
        with zipfile.ZipFile(a.output, "w", zipfile.ZIP_DEFLATED) as z:
            if a.model:
                z.write(a.model, "model/" + os.path.basename(a.model))
                manifest["model"] = os.path.basename(a.model)
            if a.data:
                base = os.path.basename(os.path.normpath(a.data))
                manifest["dataset"] = base
                if os.path.isdir(a.data):
                    for r, _, fs in os.walk(a.data):
                        for f in fs:
                            full = os.path.join(r, f)
                            z.write(full, "dataset/" + base + "/" + os.path.relpath(full, a.data))
                else:
                    z.write(a.data, "dataset/" + base)
            if a.include_config:
                for cfg in ("axonml.toml", "Axonml.toml"):
                    if os.path.exists(cfg):
                        z.write(cfg, "config/" + cfg)
                        manifest["config"].append(cfg)
            z.writestr("manifest.json", json.dumps(manifest, indent=1))
        print(f"created {a.output} ({os.path.getsize(a.output):,} bytes)")
    elif a.action == "extract":
        out = a.output or "."
        with zipfile.ZipFile(a.input) as z:
            for n in z.namelist():
                target = os.path.realpath(os.path.join(out, n))
                if not target.startswith(os.path.realpath(out) + os.sep) and target != os.path.realpath(out):
                    raise SystemExit(f"refusing to extract {n!r} outside {out}")
            z.extractall(out)
            if a.verbose:
                for n in z.namelist():
                    print(" ", n)
            print(f"extracted {len(z.namelist())} files to {out}")
    elif a.action == "list":
        with zipfile.ZipFile(a.input) as z:
            for i in z.infolist():
                print(f"{i.file_size:>12,}  {i.compress_size:>12,}  {i.filename}" if a.detailed else i.filename)


# ----------------------------------------------------------------------------- rename
def cmd_rename(a) -> None:
    src = a.path
    if not os.path.exists(src):
        raise SystemExit(f"no such {'file' if a.kind == 'model' else 'dataset'}: {src}")
    ext = os.path.splitext(src)[1] if (a.kind == "model" and os.path.isfile(src)) else ""
    new = a.new_name if a.new_name.endswith(ext) else a.new_name + ext
    dst = os.path.join(os.path.dirname(src), new)
    if os.path.exists(dst):
        if not a.force:
            raise SystemExit(f"{dst} exists (use --force)")
        (shutil.rmtree if os.path.isdir(dst) else os.remove)(dst)
    os.rename(src, dst)
    for side in (".meta.json",):
        if os.path.exists(src + side):
            os.rename(src + side, dst + side)
    ws = _ws_load()
    for key in ("model", "dataset"):
        if ws.get(key) and os.path.abspath(ws[key]["path"]) == os.path.abspath(src):
            ws[key]["path"], ws[key]["name"] = os.path.abspath(dst), os.path.splitext(new)[0]
            _ws_save(ws)
    print(f"renamed {src} -> {dst}")


# ----------------------------------------------------------------------------- load / analyze
def cmd_load(a) -> None:
    ws = _ws_load()
    if a.action == "status":
        for key in ("model", "dataset"):
            e = ws.get(key)
            print(f"{key:8s} " + (f"{e['name']}  ({e['path']})  {e.get('detail', '')}" if e else "(none)"))
        return
    if a.action == "clear":
        _ws_save({"model": None, "dataset": None})
        print("workspace cleared")
        return
    if a.action in ("model", "both"):
        path = a.path if a.action == "model" else a.model
        s = model_summary(path)
        ws["model"] = {"name": (a.name if a.action == "model" else None) or os.path.splitext(os.path.basename(path))[0],
                       "path": s["path"], "format": getattr(a, "format", None) or s["format"],
                       "detail": f"{s['parameters']:,} parameters"}
        print(f"loaded model {ws['model']['name']}: {ws['model']['detail']}")
    if a.action in ("data", "both"):
        from ..data.analysis import analyze_dataset
        path = a.path if a.action == "data" else a.data
        an = analyze_dataset(path, getattr(a, "type", None))
        ws["dataset"] = {"name": (a.name if a.action == "data" else None) or os.path.basename(os.path.normpath(path)),
                         "path": an["path"], "type": an["dataset_type"],
                         "detail": f"{an.get('num_samples')} samples, {an.get('num_classes')} classes"}
        print(f"loaded dataset {ws['dataset']['name']}: {ws['dataset']['detail']}")
    _ws_save(ws)


def compatibility(model: dict, data: dict) -> dict:
    """Does the first layer's fan-in match the dataset's feature count, and the last layer's
    fan-out its class count?"""
    two_d = [e for e in model["entries"] if len(e["shape"]) == 2]
    issues = []
    fan_in = two_d[0]["shape"][1] if two_d else None
    fan_out = two_d[-1]["shape"][0] if two_d else None
    feats = data.get("num_features")
    if data.get("image_shape"):
        feats = 1
        for s in data["image_shape"]:
            feats *= s
    if fan_in and feats and fan_in != feats and not any(len(e["shape"]) == 4 for e in model["entries"]):
        issues.append(f"model expects {fan_in} input features, dataset has {feats}")
    if fan_out and data.get("num_classes") and fan_out != data["num_classes"]:
        issues.append(f"model has {fan_out} outputs, dataset has {data['num_classes']} classes")
    return {"compatible": not issues, "issues": issues, "model_inputs": fan_in, "model_outputs": fan_out,
            "dataset_features": feats, "dataset_classes": data.get("num_classes")}


def cmd_analyze(a) -> None:
    from ..data.analysis import analyze_dataset
    ws = _ws_load()

    def model_path():
        p = getattr(a, "path_opt", None) or getattr(a, "path", None) or (ws["model"]["path"] if ws.get("model") else None)
        if not p:
            raise SystemExit("no model given and none loaded (axonml load model <path>)")
        return p

    def data_path():
        p = getattr(a, "path_opt", None) or getattr(a, "path", None) or (ws["dataset"]["path"] if ws.get("dataset") else None)
        if not p:
            raise SystemExit("no dataset given and none loaded (axonml load data <path>)")
        return p

    if a.action == "model":
        s = model_summary(model_path())
        if a.format == "json" or a.output:
            if not a.detailed:
                s = {k: v for k, v in s.items() if k != "entries"}
            _emit(s, a.format, a.output)
        else:
            _print_model(s, a.detailed)
    elif a.action == "data":
        an = analyze_dataset(data_path(), None, a.max_samples)
        if not a.detailed:
            an.pop("columns", None)
        _emit(an, a.format, a.output)
    elif a.action in ("both", "report"):
        if not (ws.get("model") and ws.get("dataset")):
            raise SystemExit("load a model and a dataset first (axonml load both --model … --data …)")
        m = model_summary(ws["model"]["path"])
        d = analyze_dataset(ws["dataset"]["path"])
        rep = {"model": {k: v for k, v in m.items() if k != "entries"}, "dataset": {k: v for k, v in d.items() if k != "columns"},
               "compatibility": compatibility(m, d)}
        fmt = getattr(a, "format", "text")
        if a.action == "report" and fmt in ("html", "md"):
            body = _as_text(rep)
            text = (f"<html><body><h1>AxonML analysis report</h1><pre>{body}</pre></body></html>" if fmt == "html"
                    else "# AxonML analysis report\n\n```\n" + body + "\n```\n")
            with open(a.output or f"analysis_report.{fmt}", "w") as f:
                f.write(text)
            print(f"wrote {a.output or 'analysis_report.' + fmt}")
        else:
            _emit(rep, "json" if fmt == "json" else "text", a.output)


# ----------------------------------------------------------------------------- parser wiring
def add_parsers(sub) -> None:
    p = sub.add_parser("upload", help="copy a model file into the workspace's model directory")
    p.add_argument("path"); p.add_argument("-n", "--name"); p.add_argument("-d", "--description"); p.add_argument("-f", "--format")
    p.add_argument("--version"); p.add_argument("-o", "--output", "--dest", dest="dest"); p.add_argument("--validate", action="store_true")
    p.add_argument("--overwrite", action="store_true"); p.add_argument("--inspect", "--info", dest="info", action="store_true")
    p.set_defaults(fn=cmd_upload)

    p = sub.add_parser("data", help="upload, analyse, list, preview and validate datasets")
    s = p.add_subparsers(dest="action", required=True)
    q = s.add_parser("upload"); q.add_argument("path"); q.add_argument("-n", "--name"); q.add_argument("-t", "--data-type", "--type", dest="type"); q.add_argument("--task")
    q.add_argument("-o", "--output", "--dest", dest="dest"); q.add_argument("--split", default="0.8,0.1,0.1"); q.add_argument("--analyze", action="store_true")
    q = s.add_parser("analyze"); q.add_argument("path"); q.add_argument("-t", "--data-type", "--type", dest="type"); q.add_argument("--max-samples", type=int, default=10000)
    q.add_argument("-f", "--format", default="text", choices=["text", "json"]); q.add_argument("-o", "--output")
    q.add_argument("--detailed", action="store_true"); q.add_argument("--recommend", action="store_true")
    q = s.add_parser("list"); q.add_argument("-p", "--path"); q.add_argument("-d", "--detailed", action="store_true")
    q = s.add_parser("config"); q.add_argument("path"); q.add_argument("-o", "--output"); q.add_argument("-f", "--format", default="toml")
    q = s.add_parser("preview"); q.add_argument("path"); q.add_argument("-n", "--num-samples", type=int, default=5)
    q.add_argument("--random", action="store_true")
    q = s.add_parser("validate"); q.add_argument("path"); q.add_argument("--num-classes", type=int); q.add_argument("--input-shape")
    q.add_argument("--check-missing", action="store_true", default=True); q.add_argument("--check-balance", action="store_true", default=True)
    p.set_defaults(fn=cmd_data)

    p = sub.add_parser("scaffold", help="generate a training project")
    s = p.add_subparsers(dest="action", required=True)
    q = s.add_parser("generate"); q.add_argument("name"); q.add_argument("-o", "--output"); q.add_argument("-t", "--template", default="training")
    q.add_argument("--task", default="classification"); q.add_argument("--architecture", "--arch", dest="arch", default="mlp")
    q.add_argument("-m", "--model", help="model file the generated project starts from"); q.add_argument("-d", "--data", help="dataset path written into the project file")
    q.add_argument("--wandb", action="store_true"); q.add_argument("--augmentation", "--augment", dest="augment", action="store_true")
    q.add_argument("--overwrite", action="store_true")
    q = s.add_parser("templates"); q.add_argument("-d", "--detailed", action="store_true")
    p.set_defaults(fn=cmd_scaffold)

    p = sub.add_parser("zip", help="model/dataset bundles")
    s = p.add_subparsers(dest="action", required=True)
    q = s.add_parser("create"); q.add_argument("output", nargs="?"); q.add_argument("-o", "--output", dest="output_opt"); q.add_argument("-m", "--model"); q.add_argument("-d", "--data")
    q.add_argument("--include-config", action="store_true"); q.add_argument("--overwrite", action="store_true")
    q = s.add_parser("extract"); q.add_argument("input"); q.add_argument("-o", "--output"); q.add_argument("-v", "--verbose", action="store_true")
    q = s.add_parser("list"); q.add_argument("input"); q.add_argument("-d", "--detailed", action="store_true")
    p.set_defaults(fn=cmd_zip)

    p = sub.add_parser("rename", help="rename a model file or a dataset")
    s = p.add_subparsers(dest="kind", required=True)
    for kind in ("model", "data"):
        q = s.add_parser(kind); q.add_argument("path"); q.add_argument("new_name"); q.add_argument("-f", "--force", action="store_true")
    p.set_defaults(fn=cmd_rename)

    p = sub.add_parser("load", help="load a model and/or dataset into the workspace")
    s = p.add_subparsers(dest="action", required=True)
    q = s.add_parser("model"); q.add_argument("path"); q.add_argument("-n", "--name"); q.add_argument("-f", "--format")
    q = s.add_parser("data"); q.add_argument("path"); q.add_argument("-n", "--name"); q.add_argument("-t", "--data-type", "--type", dest="type")
    q = s.add_parser("both"); q.add_argument("-m", "--model", required=True); q.add_argument("-d", "--data", required=True)
    s.add_parser("status"); s.add_parser("clear")
    p.set_defaults(fn=cmd_load)

    p = sub.add_parser("analyze", help="analyse the loaded (or a given) model / dataset")
    s = p.add_subparsers(dest="action", required=True)
    q = s.add_parser("model"); q.add_argument("path", nargs="?"); q.add_argument("-p", "--path", dest="path_opt"); q.add_argument("-d", "--detailed", action="store_true")
    q.add_argument("-o", "--output"); q.add_argument("-f", "--format", default="text", choices=["text", "json"])
    q = s.add_parser("data"); q.add_argument("path", nargs="?"); q.add_argument("-p", "--path", dest="path_opt"); q.add_argument("-d", "--detailed", action="store_true")
    q.add_argument("--max-samples", type=int, default=10000); q.add_argument("-o", "--output")
    q.add_argument("-f", "--format", default="text", choices=["text", "json"])
    q = s.add_parser("both"); q.add_argument("-o", "--output")
    q = s.add_parser("report"); q.add_argument("-o", "--output"); q.add_argument("-f", "--format", default="text", choices=["html", "json", "md", "text"])
    q.add_argument("--visualize", "--visualizations", dest="visualizations", action="store_true")
    p.set_defaults(fn=cmd_analyze)
