"""``axonml`` command line (``python -m axonml_b200.cli``): the subcommands of the reference's clap
CLI (crates/axonml-cli/src/cli.rs:44-145) in the reference's argument syntax, plus a distributed
launcher.  The older spellings of this package (``--checkpoint``, ``quant IN OUT``) still parse.

    new NAME [-t TEMPLATE] [--no-git]     scaffold a project directory (git-initialised)
    init [-n NAME]                        an ``axonml.toml`` in an existing directory
    train [CONFIG] [-d DATA] [-f FORMAT]  train MLP | SimpleCNN | LeNet | ResNet-18 from the project file;
                                          per-epoch ``.axonml`` checkpoints and ``training_log.jsonl``
    resume CHECKPOINT                     continue from a checkpoint (model + optimizer + training state)
    eval MODEL DATA                       loss / accuracy / per-class metrics of a model file on a dataset
    predict MODEL INPUT [-t K]            top-k classes of one sample (file, JSON list or comma list)
    report MODEL -d DATA [-f html|json|text]   evaluation report with confusion matrix and loss curves;
                                          without a model file: summary of the checkpoints in a directory
    convert IN OUT [--from F --to F]      StateDict <-> SafeTensors <-> JSON <-> PyTorch-named <-> ONNX
    export MODEL OUTPUT [-f FORMAT]       onnx | safetensors | json | axonml | gguf
    inspect MODEL [-d] [--show-params]    tensors, shapes and parameter count of a checkpoint or GGUF file
    quant convert | info | benchmark | list    real block quantisation into GGUF (Q8_0/Q4_0/Q4_1/Q5_0/Q5_1/
                                          Q4_K); ``--fake`` reproduces the reference's quantise->dequantise
                                          f32 round trip (commands/quant.rs:244-330)
    bench model | inference | compare | hardware   latency / throughput sweeps, GEMM + copy bandwidth
    gpu list | info | select | bench | memory | status   devices, memory, clocks (read-only: CUDA + NVML)
    serve [MODEL]                         inference server (StateDict models and/or a GGUF LLaMA engine)
    hub list | search | info | download | cached | clear   the pretrained-weight registries and their cache
    launch                                one process per GPU on this node (rendezvous on 127.0.0.1)

The bodies of the model-file commands live in ``commands.py``; workspace and service commands in
``workspace.py`` and ``services.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import torch

from .config import ProjectConfig


# ---------------------------------------------------------------------- helpers
def _device(name: str) -> torch.device:
    if name in ("auto", ""):
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return torch.device(name)


def build_model(cfg: ProjectConfig):
    from ..vision.models.lenet import LeNet, MLP, SimpleCNN
    m = cfg.model
    arch = m.architecture.lower()
    if arch == "mlp":
        n_in = 1
        for s in m.input_size:
            n_in *= int(s)
        return MLP(n_in, list(m.hidden_sizes), m.num_classes, m.dropout)
    if arch in ("simplecnn", "cnn"):
        ch = int(m.input_size[0]) if len(m.input_size) == 3 else 1
        return SimpleCNN(ch, m.num_classes) if _accepts(SimpleCNN, 2) else SimpleCNN.new()
    if arch == "lenet":
        return LeNet.new()
    if arch in ("resnet18", "resnet34"):
        from ..vision.models import resnet
        return getattr(resnet, arch)(m.num_classes)
    raise SystemExit(f"unknown architecture {m.architecture!r}")


def _accepts(cls, n: int) -> bool:
    import inspect
    try:
        return len(inspect.signature(cls.__init__).parameters) - 1 >= n
    except (TypeError, ValueError):
        return False


def build_datasets(cfg: ProjectConfig):
    from ..data.dataset import SubsetDataset
    from ..vision import datasets as D
    d = cfg.data
    fmt = d.format.lower()
    if fmt in ("synthetic-mnist", "synthetic"):
        full = D.SyntheticMNIST(2048, cfg.training.seed)
    elif fmt == "synthetic-cifar":
        full = D.SyntheticCIFAR(2048, cfg.model.num_classes, cfg.training.seed)
    elif fmt == "mnist":
        full = D.MNIST(d.train_path, train=True)
    elif fmt in ("fashion-mnist", "fashionmnist"):
        full = D.FashionMNIST(d.train_path, train=True)
    elif fmt == "cifar10":
        full = D.CIFAR10(d.train_path, train=True)
    else:
        raise SystemExit(f"unknown data format {d.format!r}")
    n = full.len()
    n_val = int(n * d.val_split)
    idx = list(range(n))
    return SubsetDataset(full, idx[:n - n_val]), (SubsetDataset(full, idx[n - n_val:]) if n_val else None)


def build_optimizer(cfg: ProjectConfig, params):
    from .. import optim
    t, o = cfg.training, cfg.training.optimizer
    name = o.name.lower()
    if name == "sgd":
        return optim.SGD(params, t.learning_rate).momentum(o.momentum).weight_decay(o.weight_decay).nesterov(o.nesterov)
    if name == "adam":
        return optim.Adam(params, t.learning_rate, (o.beta1, o.beta2), o.eps, o.weight_decay)
    if name == "adamw":
        return optim.AdamW(params, t.learning_rate, (o.beta1, o.beta2), o.eps, o.weight_decay or 0.01)
    if name == "rmsprop":
        return optim.RMSprop(params, t.learning_rate)
    if name == "lamb":
        return optim.LAMB(params, t.learning_rate)
    raise SystemExit(f"unknown optimizer {o.name!r}")


def _checkpoint_path(out_dir: str, epoch: int) -> str:
    return os.path.join(out_dir, f"checkpoint_epoch_{epoch}.axonml")


def _latest_checkpoint(out_dir: str):
    best, path = -1, None
    if os.path.isdir(out_dir):
        for f in os.listdir(out_dir):
            if f.startswith("checkpoint_epoch_") and f.endswith(".axonml"):
                e = int(f[len("checkpoint_epoch_"):-len(".axonml")])
                if e > best:
                    best, path = e, os.path.join(out_dir, f)
    return path


def _accuracy(model, loader, dev) -> float:
    model.eval()
    hit = tot = 0
    with torch.no_grad():
        for b in loader:
            x, y = b.data.to(dev), b.targets.to(dev)
            hit += int((model(x).argmax(-1) == y).sum())
            tot += y.numel()
    model.train()
    return hit / max(tot, 1)


# ---------------------------------------------------------------------- commands
TEMPLATES = {
    "default": {},
    "mlp": {"architecture": "mlp"},
    "cnn": {"architecture": "simplecnn", "input_size": [1, 28, 28]},
    "lenet": {"architecture": "lenet", "input_size": [1, 28, 28]},
    "resnet": {"architecture": "resnet18", "input_size": [3, 32, 32], "format": "synthetic-cifar"},
}


def _git_init(directory: str) -> bool:
    import shutil
    if shutil.which("git") is None or os.path.isdir(os.path.join(directory, ".git")):
        return False
    ok = subprocess.call(["git", "init", "-q", directory], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) == 0
    if ok:
        with open(os.path.join(directory, ".gitignore"), "a") as f:
            f.write("output/\n*.axonml\n__pycache__/\n")
    return ok


def _template_config(template: str, name: str) -> ProjectConfig:
    if template not in TEMPLATES:
        raise SystemExit(f"unknown template {template!r}; available: " + ", ".join(TEMPLATES))
    cfg = ProjectConfig()
    cfg.project.name = name
    t = TEMPLATES[template]
    if "architecture" in t:
        cfg.model.architecture = t["architecture"]
    if "input_size" in t:
        cfg.model.input_size = list(t["input_size"])
    if "format" in t:
        cfg.data.format = t["format"]
    return cfg


def cmd_new(a):
    root = os.path.join(a.path, a.name) if getattr(a, "path", None) else a.name
    os.makedirs(root, exist_ok=True)
    for sub in ("data", "output", "models"):
        os.makedirs(os.path.join(root, sub), exist_ok=True)
    _template_config(getattr(a, "template", "default"), os.path.basename(os.path.abspath(root))).save(os.path.join(root, "axonml.toml"))
    git = not getattr(a, "no_git", False) and _git_init(root)
    print(f"created project {root}/ (axonml.toml, data/, output/, models/" + (", git repository" if git else "") + ")")


def cmd_init(a):
    if os.path.exists("axonml.toml") and not a.force:
        raise SystemExit("axonml.toml exists (use --force)")
    _template_config("default", getattr(a, "name", None) or os.path.basename(os.getcwd())).save("axonml.toml")
    git = not getattr(a, "no_git", True) and _git_init(".")
    print("wrote axonml.toml" + (" and initialised a git repository" if git else ""))


def _apply_overrides(cfg: ProjectConfig, a) -> ProjectConfig:
    t = cfg.training
    for flag, attr in (("epochs", "epochs"), ("batch_size", "batch_size"), ("lr", "learning_rate"),
                       ("device", "device"), ("output", "output_dir"), ("seed", "seed")):
        v = getattr(a, flag, None)
        if v is not None:
            setattr(t, attr, v)
    if getattr(a, "optimizer", None):
        t.optimizer.name = a.optimizer
    if getattr(a, "model", None):
        cfg.model.architecture = a.model
    if getattr(a, "data", None):
        if os.path.exists(a.data):                  # the reference's form: a path, its format given or detected
            from .commands import detect_data_format
            cfg.data.train_path = a.data
            fmt = getattr(a, "format", None) or detect_data_format(a.data)
            if fmt:
                cfg.data.format = fmt
        else:
            cfg.data.format = a.data
    elif getattr(a, "format", None) and getattr(a, "cmd", "") in ("train", "resume"):
        cfg.data.format = a.format
    if getattr(a, "workers", None) is not None:
        t.num_workers = a.workers
    if getattr(a, "device", None) in (None, "auto"):
        from .commands import gpu_selected
        if gpu_selected() and t.device == "auto":
            t.device = gpu_selected()
    return cfg


def cmd_train(a, resume_from: str | None = None):
    from .. import nn
    from ..data import DataLoader
    from ..serialize import load_checkpoint, save_checkpoint
    from ..serialize.checkpoint import Checkpoint, TrainingState, optimizer_from_state_dict, optimizer_to_state_dict
    from ..serialize.state_dict import StateDict
    cfg = _apply_overrides(ProjectConfig.resolve(a.config), a)
    errs = cfg.validate()
    if errs:
        raise SystemExit("invalid configuration:\n  " + "\n  ".join(errs))
    t = cfg.training
    torch.manual_seed(t.seed)
    dev = _device(t.device)
    model = build_model(cfg).to(dev)
    opt = build_optimizer(cfg, list(model.parameters()))
    train_ds, val_ds = build_datasets(cfg)
    loader = DataLoader(train_ds, t.batch_size, shuffle=cfg.data.shuffle, num_workers=t.num_workers)
    val_loader = DataLoader(val_ds, t.batch_size) if val_ds is not None else None
    crit = nn.CrossEntropyLoss()
    os.makedirs(t.output_dir, exist_ok=True)
    state = TrainingState()
    start_epoch = 0
    if resume_from:
        ck = load_checkpoint(resume_from)
        ck.model_state.load_into(model, strict=False)
        optimizer_from_state_dict(opt, ck.optimizer_state)
        state = ck.training_state
        start_epoch = state.epoch
        print(f"resumed from {resume_from} (epoch {start_epoch}, step {state.global_step})")
    from ..integrations.wandb import WandbConfig, init_training_run
    wb = init_training_run(WandbConfig.load(), cfg.project.name, {"epochs": t.epochs, "batch_size": t.batch_size,
                                                                  "learning_rate": t.learning_rate, "optimizer": t.optimizer.name,
                                                                  "architecture": cfg.model.architecture},
                           directory=os.path.join(t.output_dir, "wandb"))
    # one JSON object per line: the run's configuration first, then one line per epoch; the terminal
    # interface follows this file (axonml tui --watch <output_dir>/training_log.jsonl)
    log = open(os.path.join(t.output_dir, "training_log.jsonl"), "a" if resume_from else "w", buffering=1)
    log.write(json.dumps({"model_name": cfg.model.architecture, "total_epochs": t.epochs, "batch_size": t.batch_size,
                          "optimizer": t.optimizer.name, "total_batches": len(loader)}) + "\n")
    for epoch in range(start_epoch, t.epochs):
        t0, losses = time.time(), []
        for b in loader:
            x, y = b.data.to(dev), b.targets.to(dev)
            opt.zero_grad()
            loss = crit(model(x), y)
            loss.backward()
            if t.gradient_clip > 0:
                from ..optim import clip_grad_norm
                clip_grad_norm(list(model.parameters()), t.gradient_clip)
            opt.step()
            losses.append(float(loss.detach()))
            state.global_step += 1
        state.epoch = epoch + 1
        mean = sum(losses) / max(len(losses), 1)
        acc = _accuracy(model, val_loader, dev) if val_loader is not None else float("nan")
        print(f"epoch {epoch + 1}/{t.epochs}  loss {mean:.4f}  val_acc {acc:.4f}  {time.time() - t0:.1f}s", flush=True)
        if wb is not None:
            wb.log_at_step(epoch + 1, {"train_loss": mean, **({} if acc != acc else {"val_accuracy": acc})})
        log.write(json.dumps({"epoch": epoch + 1, "train_loss": mean, **({} if acc != acc else {"val_acc": acc}),
                              "learning_rate": opt.get_lr(), "duration_secs": time.time() - t0}) + "\n")
        if t.checkpoint_frequency and (epoch + 1) % t.checkpoint_frequency == 0:
            ck = (Checkpoint.builder().model_state(StateDict.from_module(model))
                  .optimizer_state(optimizer_to_state_dict(opt)).training_state(state)
                  .config("architecture", cfg.model.architecture).config("val_acc", acc).build())
            save_checkpoint(ck, _checkpoint_path(t.output_dir, epoch + 1))
    log.write(json.dumps({"status": "completed"}) + "\n")
    log.close()
    if wb is not None:
        print(f"W&B offline run: {wb.finish()}")
    print(f"done: {t.output_dir}")


def cmd_resume(a):
    cfg = ProjectConfig.resolve(a.config)
    path = getattr(a, "checkpoint_pos", None) or a.checkpoint or _latest_checkpoint(a.output or cfg.training.output_dir)
    if not path:
        raise SystemExit("no checkpoint found")
    cmd_train(a, resume_from=path)


def _load_model_for(a):
    from ..serialize import load_checkpoint, load_state_dict
    cfg = _apply_overrides(ProjectConfig.resolve(a.config), a)
    model = build_model(cfg)
    path = a.checkpoint
    if path.endswith(".axonml"):
        try:
            sd = load_checkpoint(path).model_state
        except Exception:
            sd = load_state_dict(path)
    else:
        sd = load_state_dict(path)
    sd.load_into(model, strict=False)
    return cfg, model


def _write_or_print(text: str, output) -> None:
    if output:
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        with open(output, "w") as f:
            f.write(text)
        print(f"wrote {output}")
    else:
        print(text)


def cmd_eval(a):
    """``eval MODEL DATA [--format F] [-b N] [--metrics accuracy,loss,f1,...]`` on a dataset path, or
    ``eval CHECKPOINT`` with the project's validation split."""
    from . import commands as C
    if getattr(a, "data_pos", None):
        model, _ = C.model_from_file(a.checkpoint)
        ds = C.dataset_from_path(a.data_pos, a.format)
        conf, loss = C.evaluate(model, ds, a.batch_size or 32, a.device or "cpu")
        m = C.classification_metrics(conf, getattr(ds, "class_names_", None), loss)
        want = [w.strip().lower() for w in (a.metrics or "accuracy").split(",") if w.strip()]
        alias = {"f1": "macro_f1", "precision": "macro_precision", "recall": "macro_recall"}
        out = {"model": a.checkpoint, "samples": m["total_samples"]}
        for w in want:
            k = alias.get(w, w)
            if k not in m:
                raise SystemExit(f"unknown metric {w!r}; available: accuracy, loss, precision, recall, f1, weighted_f1, confusion_matrix, per_class")
            out[w] = m[k]
        _write_or_print(json.dumps(out), a.output)
        return
    from ..data import DataLoader
    cfg, model = _load_model_for(a)
    dev = _device(cfg.training.device)
    _, val = build_datasets(cfg)
    if val is None:
        raise SystemExit("no validation split configured")
    acc = _accuracy(model.to(dev), DataLoader(val, a.batch_size or cfg.training.batch_size), dev)
    print(json.dumps({"checkpoint": a.checkpoint, "samples": val.len(), "accuracy": acc}))


def cmd_predict(a):
    """``predict MODEL INPUT`` (a file, a JSON array or comma-separated numbers) or, with the
    project's data, ``predict CHECKPOINT --index N``."""
    if getattr(a, "input", None):
        from . import commands as C
        model, arch = C.model_from_file(a.checkpoint)
        x = C.shape_input_for(model, C.load_input(a.input))
        with torch.no_grad():
            p = torch.softmax(C._feed(model.to(a.device or "cpu"), x.to(a.device or "cpu")).float(), -1).cpu()
        rows = []
        for i in range(p.shape[0]):
            r = {"sample": i, "predicted": int(p[i].argmax()), "confidence": float(p[i].max())}
            if a.top_k:
                top = torch.topk(p[i], min(a.top_k, p.shape[1]))
                r["top_k"] = [{"class": int(c), "probability": float(v)} for v, c in zip(top.values, top.indices)]
            rows.append(r)
        fmt = (a.format or "json").lower()
        if fmt == "json":
            text = json.dumps({"model": a.checkpoint, "architecture": arch, "predictions": rows})
        elif fmt == "csv":
            text = "sample,predicted,confidence\n" + "\n".join(f"{r['sample']},{r['predicted']},{r['confidence']:.6f}" for r in rows)
        else:
            text = "\n".join(f"sample {r['sample']}: class {r['predicted']} ({100 * r['confidence']:.1f}%)" for r in rows)
        _write_or_print(text, a.output)
        return
    cfg, model = _load_model_for(a)
    _, val = build_datasets(cfg)
    x, y = val.get(a.index)
    model.eval()
    with torch.no_grad():
        p = torch.softmax(model(x.unsqueeze(0)).float(), -1)[0]
    print(json.dumps({"index": a.index, "label": int(y), "predicted": int(p.argmax()), "confidence": float(p.max())}))


def cmd_convert(a):
    from ..serialize import load_state_dict, save_state_dict
    from ..serialize.convert import from_pytorch_state_dict, to_pytorch_state_dict
    from ..serialize.format import Format, detect_format
    src_fmt = (getattr(a, "from_", None) or "").lower()
    if src_fmt in ("pytorch", "torch", "pt", "pth") or a.input.endswith((".pt", ".pth")):
        raw = torch.load(a.input, map_location="cpu", weights_only=True)
        raw = raw.get("state_dict", raw.get("model_state_dict", raw)) if isinstance(raw, dict) else raw
        sd = from_pytorch_state_dict({k: v for k, v in raw.items() if torch.is_tensor(v)})
    else:
        sd = load_state_dict(a.input)
    dst_fmt = (getattr(a, "to", None) or "").lower()
    if dst_fmt in ("pytorch", "torch", "pt", "pth") or a.output.endswith((".pt", ".pth")):
        torch.save(to_pytorch_state_dict(sd), a.output)
        print(f"{a.input} -> {a.output} ({len(list(sd.keys()))} tensors, PyTorch state dict)")
        return
    if dst_fmt == "onnx" or a.output.endswith(".onnx"):
        from ..onnx.export import export_module, export_onnx
        from . import commands as C
        model, _ = C.model_from_file(a.input)
        export_onnx(export_module(model, list(C.example_input(model, 1, "cpu").shape), os.path.basename(a.input)), a.output)
        print(f"{a.input} -> {a.output} (ONNX)")
        return
    if getattr(a, "optimize", False):
        # drop what inference does not need: optimizer-only buffers and batch counters
        from ..serialize.state_dict import StateDict
        keep = {k: v for k, v in sd.to_tensors().items() if not k.endswith("num_batches_tracked")}
        sd = StateDict.from_tensors({k: v.contiguous() for k, v in keep.items()})
    if a.pytorch_keys == "to":
        from ..serialize.state_dict import StateDict
        sd = StateDict.from_tensors(to_pytorch_state_dict(sd))
    elif a.pytorch_keys == "from":
        sd = from_pytorch_state_dict(sd.to_tensors())
    named = {"axonml": Format.Axonml, "json": Format.Json, "safetensors": Format.SafeTensors, "gguf": Format.Gguf}
    save_state_dict(sd, a.output, Format[a.format] if a.format else named.get(dst_fmt) or detect_format(a.output))
    print(f"{a.input} -> {a.output} ({len(list(sd.keys()))} tensors)")


def cmd_export(a):
    """``export MODEL OUTPUT [-f onnx|safetensors|json|gguf] [--quantize] [--precision fp16|bf16|fp32|q8_0|...]``;
    the earlier form ``export OUT.onnx --checkpoint CK`` still works."""
    from ..onnx.export import export_module, export_onnx
    if getattr(a, "output_pos", None) is None:
        cfg, model = _load_model_for(a) if a.checkpoint else (_apply_overrides(ProjectConfig.resolve(a.config), a), None)
        if model is None:
            model = build_model(cfg)
        shape = [1] + [int(s) for s in cfg.model.input_size]
        if cfg.model.architecture.lower() in ("lenet", "simplecnn", "cnn"):
            shape = [1, 1, 28, 28]
        export_onnx(export_module(model, shape, cfg.project.name), a.onnx_path)
        print(f"wrote {a.onnx_path}")
        return
    from . import commands as C
    src, dst, fmt = a.onnx_path, a.output_pos, (a.format or "onnx").lower()
    model, arch = C.model_from_file(src)
    if fmt == "onnx":
        export_onnx(export_module(model, list(C.example_input(model, 1, "cpu").shape), os.path.splitext(os.path.basename(src))[0]), dst)
    else:
        from ..serialize import save_state_dict
        from ..serialize.state_dict import StateDict
        prec = (a.precision or "fp16").lower()
        tensors = {k: v.detach() for k, v in model.state_dict().items()}
        if fmt == "gguf" or (a.quantize and prec.startswith("q")):
            from ..quant.gguf import write_gguf
            from ..quant.quantize import quantize_tensor
            qt = C.quant_type(prec if prec.startswith("q") else "q8_0") if a.quantize else None
            out = {k: (quantize_tensor(v.float(), qt) if qt and v.dim() >= 2 and v.shape[-1] % qt.block_size() == 0 else v.float())
                   for k, v in tensors.items()}
            write_gguf(dst, out, {"general.name": os.path.basename(src), "general.architecture": arch})
        else:
            if a.quantize:
                dt = {"fp16": torch.float16, "f16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}.get(prec)
                if dt is None:
                    raise SystemExit(f"--precision {prec} needs --format gguf")
                tensors = {k: (v.to(dt) if v.is_floating_point() else v) for k, v in tensors.items()}
            from ..serialize.format import Format
            named = {"safetensors": Format.SafeTensors, "json": Format.Json, "axonml": Format.Axonml}
            if fmt not in named:
                raise SystemExit(f"unknown export format {fmt!r}; available: onnx, safetensors, json, axonml, gguf")
            if fmt == "safetensors":                  # keeps the chosen storage precision
                from ..serialize.codec import safetensors_dumps
                with open(dst, "wb") as f:
                    f.write(safetensors_dumps({k: v.contiguous() for k, v in tensors.items()}, {"architecture": arch, "format": "pt"}))
            else:
                save_state_dict(StateDict.from_tensors({k: v.float() for k, v in tensors.items()}), dst, named[fmt])
    print(f"exported {src} ({arch}) -> {dst} [{fmt}, target {a.target or 'cpu'}]")


def cmd_inspect(a):
    """``inspect MODEL [-d] [--show-params N] [-f text|json]``."""
    from .workspace import model_summary
    s = model_summary(a.path)
    epoch = None
    if s["format"] not in ("gguf", "onnx"):
        try:
            from ..serialize import load_checkpoint
            ck = load_checkpoint(a.path)
            epoch = {"epoch": ck.epoch(), "step": ck.global_step(), "version": ck.axonml_version, "config": ck.config}
        except Exception:  # noqa: BLE001 - not a checkpoint container
            pass
    if (getattr(a, "format", None) or "text").lower() == "json":
        out = {k: s[k] for k in ("path", "format", "file_bytes", "tensors", "parameters")}
        out["checkpoint"] = epoch
        out["layers"] = s["layers"]
        if getattr(a, "detailed", False):
            out["entries"] = s["entries"]
        print(json.dumps(out, indent=1))
        return
    if epoch:
        print(f"checkpoint: epoch {epoch['epoch']} step {epoch['step']} version {epoch['version']} config {epoch['config']}")
    if s["format"] == "gguf":
        from ..quant.gguf import read_gguf
        print(f"metadata keys: {len(read_gguf(a.path).metadata)}")
    for r in s["entries"]:
        print(f"{r['name']:60s} {str(tuple(r['shape'])):24s} {r['dtype']}")
    if getattr(a, "detailed", False):
        print("layers:")
        for l in s["layers"]:
            print(f"  {l['name']:56s} {l['parameters']:>12,d}")
    n = getattr(a, "show_params", None)
    if n and s["format"] not in ("gguf", "onnx"):
        from .commands import _state_of
        for k, v in _state_of(a.path)[0].to_tensors().items():
            vals = ", ".join(f"{x:.4g}" for x in v.flatten()[:n].float().tolist())
            print(f"{k}: [{vals}{', ...' if v.numel() > n else ''}]")
    print(f"{s['parameters']:,} parameters in {s['tensors']} tensors, {s['file_bytes']:,} bytes ({s['format']})")


def cmd_quant_info(a):
    from .commands import quant_info
    info = quant_info(a.input, a.detailed)
    print(json.dumps(info, indent=1))


def cmd_quant_benchmark(a):
    from .commands import QUANT_TYPES, quant_benchmark
    types = [t.strip() for t in a.types.split(",")] if a.types else [n for n, _, _ in QUANT_TYPES if n.startswith("q")]
    print(json.dumps({"model": a.input, "iterations": a.iterations, "results": quant_benchmark(a.input, types, a.iterations)}, indent=1))


def cmd_quant_list(a):
    from .commands import QUANT_TYPES
    for name, desc, bits in QUANT_TYPES:
        print(f"{name:6s} {bits:5.1f} bits/value  {desc}")


def cmd_quant(a):
    """``quant convert INPUT -t TYPE -o OUTPUT`` (GGUF with real blocks; ``--fake`` writes the
    quantise -> dequantise round trip as an f32 state dict, which is what the reference's convert does)."""
    from ..quant.quantize import compute_quantization_error, dequantize_tensor, quantize_tensor
    from ..serialize import save_state_dict
    from .commands import _state_of, quant_type
    if getattr(a, "target", None):
        a.type = a.target
    if getattr(a, "output_opt", None):
        a.output = a.output_opt
    if not getattr(a, "output", None):
        raise SystemExit("quant convert needs an output path (-o)")
    if os.path.exists(a.output) and getattr(a, "overwrite", None) is False and getattr(a, "target", None):
        raise SystemExit(f"{a.output} exists (use --overwrite)")
    qt = quant_type(a.type)
    sd = _state_of(a.input)[0]
    if a.fake:
        from ..serialize.state_dict import StateDict
        out, errs = {}, []
        for k, v in sd.to_tensors().items():
            if v.numel() >= a.min_numel and v.dim() >= 2 and v.shape[-1] % qt.block_size() == 0:
                d = dequantize_tensor(quantize_tensor(v.float(), qt)).view_as(v)
                errs.append(compute_quantization_error(v.float(), d))
                v = d
            out[k] = v
        save_state_dict(StateDict.from_tensors(out), a.output)
        print(f"fake-quantised {len(errs)} tensors to {qt.name}, mean rmse {sum(errs) / max(len(errs), 1):.3e} -> {a.output}")
        return
    from ..quant.gguf import write_gguf
    plain, quant = {}, {}
    for k, v in sd.to_tensors().items():
        if v.numel() >= a.min_numel and v.dim() >= 2 and v.shape[-1] % qt.block_size() == 0:
            quant[k] = quantize_tensor(v.float(), qt)
        else:
            plain[k] = v.float()
    nq = len(quant)
    write_gguf(a.output, {**plain, **quant}, {"general.name": os.path.basename(a.input), "general.quantization": qt.name})
    print(f"quantised {nq} tensors to {qt.name} -> {a.output} ({os.path.getsize(a.output):,} bytes)")


def cmd_bench(a):
    """``bench model INPUT`` | ``bench inference MODEL -b 1,8,32`` | ``bench compare A,B`` | ``bench hardware``;
    ``bench model`` without a file benchmarks the project's configured model over ``--batch-sizes``."""
    from .. import benchmark as B
    from . import commands as C
    what, target = a.what, getattr(a, "target", None)
    dev_name = a.device or "auto"
    csv = [int(x) for x in str(a.batch_size or "").replace(" ", ",").split(",") if x]
    a.batch_size, a.batch_sizes_csv = (csv[0] if csv else None), (",".join(map(str, csv)) if len(csv) > 1 or what == "inference" and csv else None)
    if what in ("inference", "compare") and not target:
        raise SystemExit(f"bench {what} needs a model file")
    if what == "model" and target:
        out = C.bench_model_file(target, a.iterations, a.warmup, a.batch_size or 1, dev_name)
        _write_or_print(json.dumps(out), a.output)
        return
    if what == "inference":
        sizes = [int(x) for x in str(a.batch_sizes_csv or "1,8,32").replace(" ", ",").split(",") if x]
        rows = [C.bench_model_file(target, a.iterations, a.warmup, bs, dev_name) for bs in sizes]
        _write_or_print(json.dumps({"model": target, "results": rows}), a.output)
        return
    if what == "compare":
        rows = [C.bench_model_file(m.strip(), a.iterations, a.warmup, a.batch_size or 1, dev_name) for m in target.split(",") if m.strip()]
        best = min(rows, key=lambda r: r["mean_ms"])
        for r in rows:
            r["relative"] = r["mean_ms"] / best["mean_ms"]
        _write_or_print(json.dumps({"fastest": best["model"], "results": rows}), a.output)
        return
    if what == "hardware":
        dev = _device("auto")
        out = {"device": str(dev)}
        if dev.type == "cuda":
            from ..ops.gemm import gemm_bf16, gemm_supported
            n = 8192
            x = torch.randn(n, n, device=dev).bfloat16()
            y = torch.randn(n, n, device=dev).bfloat16()
            f = (lambda: gemm_bf16(x, y)) if gemm_supported(x, y) else (lambda: x @ y.t())
            for _ in range(3):
                f()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                f()
            e1.record()
            torch.cuda.synchronize()
            out["bf16_gemm_tflops"] = 2 * n ** 3 * 10 / (e0.elapsed_time(e1) / 1e3) / 1e12
            src = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
            dst = torch.empty_like(src)
            dst.copy_(src)
            e0.record()
            for _ in range(5):
                dst.copy_(src)
            e1.record()
            torch.cuda.synchronize()
            out["copy_gbs"] = 2 * src.numel() * 5 / (e0.elapsed_time(e1) / 1e3) / 1e9
        else:
            n = 512
            x, y = torch.randn(n, n), torch.randn(n, n)
            t0 = time.perf_counter()
            for _ in range(10):
                x @ y
            out["f32_matmul_gflops"] = 2 * n ** 3 * 10 / (time.perf_counter() - t0) / 1e9
        print(json.dumps(out))
        return
    cfg = _apply_overrides(ProjectConfig.resolve(a.config), a)
    dev = _device(cfg.training.device)
    model = build_model(cfg).to(dev).eval()
    shape = [1, 1, 28, 28] if cfg.model.architecture.lower() in ("lenet", "simplecnn", "cnn") else [1] + list(cfg.model.input_size)
    rows = []
    for bs in a.batch_sizes:
        x = torch.randn([bs] + shape[1:], device=dev)
        r = B.benchmark_model(model, x, iterations=a.iterations, name=f"{cfg.model.architecture}@{bs}")
        rows.append({"batch": bs, "mean_ms": r.mean_ms if hasattr(r, "mean_ms") else None,
                     "throughput": (bs / (r.mean_ms / 1e3)) if getattr(r, "mean_ms", 0) else None})
    print(json.dumps({"model": cfg.model.architecture, "device": str(dev), "results": rows}))


def cmd_gpu(a):
    """``gpu list | info | select DEV [-p] | bench [-d DEV | -a] | memory | status`` (read-only: CUDA + NVML)."""
    from . import commands as C
    action = getattr(a, "action", None) or "list"
    if action == "select":
        if not a.device_pos:
            raise SystemExit("gpu select needs a device (an index, cuda:N or cpu)")
        print(json.dumps(C.gpu_select(a.device_pos, a.persistent)))
        return
    if action == "bench":
        if not torch.cuda.is_available():
            raise SystemExit("no CUDA device to benchmark")
        idx = list(range(torch.cuda.device_count())) if a.all else [int(str(a.device or "0").split(":")[-1])]
        print(json.dumps([C.gpu_bench(i, a.iterations) for i in idx], indent=1))
        return
    if action == "memory":
        print(json.dumps([{k: d[k] for k in ("index", "name", "memory_total_bytes", "memory_free_bytes")} for d in C.gpu_devices()], indent=1))
        return
    if action == "status":
        print(json.dumps({"cuda_available": torch.cuda.is_available(), "device_count": len(C.gpu_devices()), "selected": C.gpu_selected()}))
        return
    out = {"cuda_available": torch.cuda.is_available(), "devices": []}
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        out["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                               "memory_gb": round(p.total_memory / 2 ** 30, 1)})
    try:
        import pynvml
        pynvml.nvmlInit()
        for d in out["devices"]:
            h = pynvml.nvmlDeviceGetHandleByIndex(d["index"])
            d["sm_clock_mhz"] = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
            d["power_w"] = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
            m = pynvml.nvmlDeviceGetMemoryInfo(h)
            d["memory_used_gb"] = round(m.used / 2 ** 30, 2)
        pynvml.nvmlShutdown()
    except Exception:
        pass
    out["selected"] = C.gpu_selected()
    print(json.dumps(out, indent=1))


def cmd_serve(a):
    from ..server.http import AxonmlHTTPServer
    from ..server.inference import InferenceServer
    engine = None
    if a.gguf:
        from ..server import LLMEngine, QuantizedLlama
        engine = LLMEngine(QuantizedLlama.from_gguf(a.gguf, device="cuda" if torch.cuda.is_available() else "cpu"),
                           max_batch=a.max_batch, max_context=a.max_context)
        engine.warmup()
    inf = InferenceServer()
    specs = list(a.model or [])
    if getattr(a, "model_pos", None):
        if a.model_pos.endswith(".gguf") and not a.gguf:
            raise SystemExit("pass GGUF files with --gguf")
        specs.append(f"{os.path.splitext(os.path.basename(a.model_pos))[0]}={a.model_pos}")
    a.model = specs
    for spec in specs:
        name, path = spec.split("=", 1)
        inf.load(name, path)
    srv = AxonmlHTTPServer(a.host, a.port, inf, engine)
    print(f"serving on http://{a.host}:{a.port} (models: {[s.split('=')[0] for s in a.model or []]}, llm: {bool(engine)})", flush=True)
    srv.serve_forever()


def cmd_hub(a):
    """``hub list | search Q | info M | download M [-f] | cached | clear [M]`` over the unified
    registry; weights come from the vision and language-model hubs."""
    from .. import hub
    from ..llm import hub as lhub
    from ..vision import hub as vhub

    def locate(name):
        if name in vhub.model_registry():
            return vhub
        if name in lhub.llm_registry():
            return lhub
        return None

    if a.action == "list":
        for m in hub.list_all_models():
            print(f"{m.name:28s} {m.architecture:14s} {m.num_parameters:>14,d}  {m.description}")
        print("pretrained weights:")
        for m in vhub.list_models():
            print(f"  {m.name:26s} vision  {m.size_bytes / 1e6:8.1f} MB  top-1 {m.accuracy:.2f}%" + ("  [cached]" if vhub.is_cached(m.name) else ""))
        for m in lhub.list_models():
            print(f"  {m.name:26s} {m.architecture:7s} {m.size_bytes / 1e6:8.1f} MB  {m.params_str()}" + ("  [cached]" if lhub.is_cached(m.name) else ""))
    elif a.action == "search":
        for m in hub.search_models(a.query or ""):
            print(m.name)
    elif a.action == "info":
        m = hub.get_model_info(a.query)
        h = locate(a.query)
        if m is None and h is None:
            raise SystemExit(f"unknown model {a.query!r}")
        out = {}
        if m is not None:
            out = {"name": m.name, "architecture": m.architecture, "parameters": m.num_parameters, "size_mb": m.size_mb(), "tasks": m.tasks,
                   "cached": hub.is_cached(m.name)}
        if h is not None:
            import dataclasses
            info = h.model_info(a.query)
            out.update({"name": info.name, "pretrained": dataclasses.asdict(info) | {"url": info.url}, "weights_cached": h.is_cached(a.query)})
        print(json.dumps(out))
    elif a.action == "download":
        h = locate(a.query or "")
        if h is None:
            raise SystemExit(f"no pretrained weights are registered for {a.query!r}")
        from ..hub.download import HubError
        try:
            print(h.download_weights(a.query, force=a.force))
        except HubError as e:
            raise SystemExit(str(e)) from e
    elif a.action == "cached":
        for h, kind in ((vhub, "vision"), (lhub, "llm")):
            d = h.cache_dir()
            for f in sorted(os.listdir(d)) if os.path.isdir(d) else []:
                print(f"{kind:7s} {f:40s} {os.path.getsize(os.path.join(d, f)):>14,d} bytes")
    elif a.action == "clear":
        n = 0
        for h in (vhub, lhub):
            d = h.cache_dir()
            for f in sorted(os.listdir(d)) if os.path.isdir(d) else []:
                if a.query is None or os.path.splitext(f)[0] == a.query:
                    os.remove(os.path.join(d, f))
                    n += 1
        print(f"removed {n} cached file(s)")


def cmd_launch(a):
    """One process per GPU on this node: ``axonml launch --nproc 8 script.py [args...]``."""
    n = a.nproc or max(torch.cuda.device_count(), 1)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(a.port), a.script] + a.script_args
    raise SystemExit(subprocess.call(cmd))


def cmd_report(a):
    """``report MODEL -d DATA [-f html|json|text] [-o FILE]``: evaluation report (accuracy, per-class
    precision / recall / F1, confusion matrix, loss curves from ``--history``); ``report DIR`` lists
    the checkpoints of an output directory."""
    from ..serialize import load_checkpoint
    if not os.path.isdir(a.dir):
        from . import commands as C
        if not a.data:
            raise SystemExit("report needs --data (a dataset path or synthetic-mnist / synthetic-cifar)")
        model, arch = C.model_from_file(a.dir)
        ds = C.dataset_from_path(a.data, a.dataset_format)
        conf, loss = C.evaluate(model, ds, a.batch_size, a.device, a.num_classes)
        names = [n.strip() for n in a.class_names.split(",")] if a.class_names else getattr(ds, "class_names_", None)
        if names is None and hasattr(ds, "class_names") and callable(ds.class_names):
            names = ds.class_names()
        metrics = C.classification_metrics(conf, names, loss)
        history = C.load_history(a.history or os.path.join(os.path.dirname(os.path.abspath(a.dir)), "training_log.jsonl"))
        on = lambda v: str(v).lower() not in ("false", "0", "no")
        fmt = (a.format or "html").lower()
        text = C.render_report(metrics, f"{os.path.basename(a.dir)} ({arch})", fmt, history, on(a.confusion_matrix), on(a.per_class_metrics),
                               on(a.loss_curves))
        out = a.output or (None if fmt == "text" else f"report.{fmt}")
        _write_or_print(text, out)
        if out:
            print(f"accuracy {metrics['accuracy']:.4f}  macro F1 {metrics['macro_f1']:.4f}  ({metrics['total_samples']} samples)")
        return
    rows = []
    for f in sorted(os.listdir(a.dir)):
        if f.endswith(".axonml"):
            try:
                ck = load_checkpoint(os.path.join(a.dir, f))
                rows.append({"file": f, "epoch": ck.epoch(), "step": ck.global_step(), **ck.config})
            except Exception as e:  # noqa: BLE001
                rows.append({"file": f, "error": str(e)})
    print(json.dumps(rows, indent=1))


# ---------------------------------------------------------------------- parser
def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="axonml", description="AxonML command line (B200 build)")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p, short=True):
        p.add_argument("-c", "--config", default=os.environ.get("AXONML_CONFIG"))
        p.add_argument(*(("-m",) if short else ()), "--model")
        p.add_argument("-d", "--data"); p.add_argument("--device")
        p.add_argument("-o", "--output"); p.add_argument("--seed", type=int)
        return p

    p = sub.add_parser("new", help="create a project directory"); p.add_argument("name")
    p.add_argument("-t", "--template", default="default", help="default | mlp | cnn | lenet | resnet")
    p.add_argument("--no-git", action="store_true"); p.add_argument("-p", "--path"); p.set_defaults(fn=cmd_new)
    p = sub.add_parser("init", help="write axonml.toml into this directory"); p.add_argument("-n", "--name")
    p.add_argument("--no-git", action="store_true"); p.add_argument("-f", "--force", action="store_true"); p.set_defaults(fn=cmd_init, no_git=True)
    for name, fn in (("train", cmd_train), ("resume", cmd_resume)):
        p = common(sub.add_parser(name))
        p.add_argument("-e", "--epochs", type=int); p.add_argument("-b", "--batch-size", type=int, dest="batch_size")
        p.add_argument("-l", "--lr", type=float); p.add_argument("--optimizer")
        p.add_argument("--format", help="data format: mnist | fashion-mnist | cifar10 | synthetic-mnist | synthetic-cifar")
        p.add_argument("--workers", type=int)
        if name == "resume":
            p.add_argument("checkpoint_pos", nargs="?", metavar="checkpoint"); p.add_argument("--checkpoint")
        p.set_defaults(fn=fn)
    p = common(sub.add_parser("eval"), short=False); p.add_argument("checkpoint", metavar="model"); p.add_argument("data_pos", nargs="?", metavar="data")
    p.add_argument("--format"); p.add_argument("-b", "--batch-size", type=int, dest="batch_size"); p.add_argument("-m", "--metrics", default="accuracy")
    p.set_defaults(fn=cmd_eval)
    p = common(sub.add_parser("predict")); p.add_argument("checkpoint", metavar="model"); p.add_argument("input", nargs="?")
    p.add_argument("--index", type=int, default=0); p.add_argument("-f", "--format", default="json", help="json | csv | text")
    p.add_argument("-t", "--top-k", type=int, dest="top_k"); p.set_defaults(fn=cmd_predict)
    p = sub.add_parser("convert"); p.add_argument("input"); p.add_argument("output")
    p.add_argument("--format", choices=["Axonml", "Json", "SafeTensors"]); p.add_argument("--pytorch-keys", choices=["to", "from"])
    p.add_argument("--from", dest="from_", help="source format (pytorch, safetensors, axonml, json); detected from the file otherwise")
    p.add_argument("--to", help="target format (axonml, safetensors, json, gguf, pytorch, onnx); detected from the extension otherwise")
    p.add_argument("--optimize", action="store_true", help="drop tensors inference does not use")
    p.set_defaults(fn=cmd_convert)
    p = common(sub.add_parser("export")); p.add_argument("onnx_path", metavar="model"); p.add_argument("output_pos", nargs="?", metavar="output")
    p.add_argument("--checkpoint"); p.add_argument("-f", "--format", default="onnx"); p.add_argument("--target", default="cpu")
    p.add_argument("--quantize", action="store_true"); p.add_argument("--precision", default="fp16"); p.set_defaults(fn=cmd_export)
    p = sub.add_parser("inspect"); p.add_argument("path", metavar="model"); p.add_argument("-d", "--detailed", action="store_true")
    p.add_argument("--show-params", type=int, dest="show_params"); p.add_argument("-f", "--format", default="text"); p.set_defaults(fn=cmd_inspect)

    p = sub.add_parser("quant", help="convert | info | benchmark | list")
    qs = p.add_subparsers(dest="action", required=True)
    q = qs.add_parser("convert"); q.add_argument("input"); q.add_argument("output", nargs="?")
    q.add_argument("-t", "--target"); q.add_argument("-o", "--output", dest="output_opt"); q.add_argument("--from", dest="from_")
    q.add_argument("--type", default="q8_0"); q.add_argument("--fake", action="store_true"); q.add_argument("--min-numel", type=int, default=1024)
    q.add_argument("--calibration-data"); q.add_argument("--calibration-samples", type=int, default=100); q.add_argument("--overwrite", action="store_true")
    q.set_defaults(fn=cmd_quant)
    q = qs.add_parser("info"); q.add_argument("input"); q.add_argument("-d", "--detailed", action="store_true"); q.set_defaults(fn=cmd_quant_info)
    q = qs.add_parser("benchmark"); q.add_argument("input"); q.add_argument("-i", "--iterations", type=int, default=10); q.add_argument("-t", "--types")
    q.set_defaults(fn=cmd_quant_benchmark)
    qs.add_parser("list").set_defaults(fn=cmd_quant_list)

    p = common(sub.add_parser("bench")); p.add_argument("what", choices=["model", "inference", "compare", "hardware"], nargs="?", default="model")
    p.add_argument("target", nargs="?", metavar="input", help="model file (comma-separated files for compare)")
    p.add_argument("--batch-sizes", type=int, nargs="+", default=[1, 8, 32]); p.add_argument("-i", "--iterations", type=int, default=20)
    p.add_argument("-w", "--warmup", type=int, default=5); p.add_argument("-b", "--batch-size", "--batches", dest="batch_size", help="one batch size, or for `bench inference` a comma-separated list")
    p.set_defaults(fn=cmd_bench)
    p = sub.add_parser("gpu"); p.add_argument("action", nargs="?", default="list", choices=["list", "info", "select", "bench", "memory", "status"])
    p.add_argument("device_pos", nargs="?", metavar="device"); p.add_argument("-p", "--persistent", action="store_true")
    p.add_argument("-d", "--device"); p.add_argument("-a", "--all", action="store_true"); p.add_argument("-i", "--iterations", type=int, default=10)
    p.set_defaults(fn=cmd_gpu)
    p = sub.add_parser("serve"); p.add_argument("model_pos", nargs="?", metavar="model"); p.add_argument("--host", default="127.0.0.1")
    p.add_argument("-p", "--port", type=int, default=3021)
    p.add_argument("--model", action="append", help="name=path of a StateDict model"); p.add_argument("--gguf")
    p.add_argument("--max-batch", "--max-batch-size", type=int, default=64, dest="max_batch"); p.add_argument("--max-context", type=int, default=1024)
    p.add_argument("--workers", type=int, default=4, help="accepted for compatibility: requests are served by one thread per connection")
    p.add_argument("--batch", action="store_true", help="accepted for compatibility: the LLM engine always batches")
    p.add_argument("--timeout", type=int, default=30000, help="per-request timeout in ms")
    p.set_defaults(fn=cmd_serve)
    p = sub.add_parser("hub"); p.add_argument("action", choices=["list", "search", "info", "download", "cached", "clear"]); p.add_argument("query", nargs="?", metavar="model")
    p.add_argument("-f", "--force", action="store_true"); p.set_defaults(fn=cmd_hub)
    p = sub.add_parser("launch"); p.add_argument("--nproc", type=int, default=0); p.add_argument("--port", type=int, default=29500)
    p.add_argument("script"); p.add_argument("script_args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_launch)
    p = sub.add_parser("report"); p.add_argument("dir", metavar="model"); p.add_argument("-d", "--data"); p.add_argument("--dataset-format")
    p.add_argument("-b", "--batch-size", type=int, default=32, dest="batch_size"); p.add_argument("--device", default="cpu"); p.add_argument("-o", "--output")
    p.add_argument("-f", "--format", default="html", help="html | json | text")
    p.add_argument("--confusion-matrix", nargs="?", const="true", default="true"); p.add_argument("--loss-curves", nargs="?", const="true", default="true")
    p.add_argument("--per-class-metrics", nargs="?", const="true", default="true"); p.add_argument("--num-classes", type=int)
    p.add_argument("--class-names"); p.add_argument("--history"); p.set_defaults(fn=cmd_report)
    from . import services, workspace
    workspace.add_parsers(sub)
    services.add_parsers(sub)
    return ap


_QUANT_ACTIONS = ("convert", "info", "benchmark", "list", "-h", "--help")


def _normalise(argv: list) -> list:
    """Earlier spellings that the parser no longer takes directly: ``quant IN OUT --type T`` is ``quant convert IN OUT --type T``."""
    if len(argv) >= 2 and argv[0] == "quant" and argv[1] not in _QUANT_ACTIONS:
        return ["quant", "convert"] + argv[1:]
    if argv and argv[0] == "predict" and "--" not in argv:
        # comma-separated input that starts with a negative number would be read as an option
        import re
        neg = [x for x in argv[1:] if re.match(r"^-[\d.][\d.eE+\-,; ]*$", x)]
        if len(neg) == 1:
            return [x for x in argv if x != neg[0]] + ["--", neg[0]]
    return argv


def main(argv=None) -> int:
    a = build_parser().parse_args(_normalise(list(sys.argv[1:] if argv is None else argv)))
    a.fn(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
