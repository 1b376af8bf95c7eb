"""``axonml`` command line (``python -m axonml_b200.cli``): the subcommands of the reference's clap
CLI (crates/axonml-cli/src/cli.rs:44-145) that make sense without its web services, plus a
distributed launcher.

    new / init      scaffold a project directory / an ``axonml.toml``
    train / resume  train MLP | SimpleCNN | LeNet | ResNet-18 from the project file; per-epoch ``.axonml``
                    checkpoints (model + optimizer + training state), resumable
    eval / predict  accuracy of a checkpoint on the validation split / class of one sample
    convert         StateDict <-> SafeTensors <-> JSON <-> PyTorch-named StateDict
    export          ONNX export of the configured model
    inspect         tensors, shapes and parameter count of a checkpoint or GGUF file
    quant           real block quantisation of a checkpoint into GGUF (Q8_0/Q4_0/Q4_1/Q5_0/Q5_1/Q4_K),
                    ``--fake`` reproduces the reference's quantise->dequantise f32 round trip
                    (commands/quant.rs:244-330)
    bench           model latency/throughput sweep, hardware GEMM + copy bandwidth
    gpu             devices, memory, clocks (read-only: CUDA + NVML)
    serve           inference server (StateDict models and/or a GGUF LLaMA engine)
    hub             list / search / info of the model registry
    launch          one process per GPU on this node (torch.distributed rendezvous on 127.0.0.1)
    report          summary of the checkpoints in an output directory
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
def cmd_new(a):
    os.makedirs(a.name, exist_ok=True)
    for sub in ("data", "output", "models"):
        os.makedirs(os.path.join(a.name, sub), exist_ok=True)
    cfg = ProjectConfig()
    cfg.project.name = os.path.basename(os.path.abspath(a.name))
    cfg.save(os.path.join(a.name, "axonml.toml"))
    print(f"created project {a.name}/ (axonml.toml, data/, output/, models/)")


def cmd_init(a):
    if os.path.exists("axonml.toml") and not a.force:
        raise SystemExit("axonml.toml exists (use --force)")
    ProjectConfig().save("axonml.toml")
    print("wrote axonml.toml")


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
        cfg.data.format = a.data
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
    path = a.checkpoint or _latest_checkpoint(a.output or cfg.training.output_dir)
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


def cmd_eval(a):
    from ..data import DataLoader
    cfg, model = _load_model_for(a)
    dev = _device(cfg.training.device)
    _, val = build_datasets(cfg)
    if val is None:
        raise SystemExit("no validation split configured")
    acc = _accuracy(model.to(dev), DataLoader(val, cfg.training.batch_size), dev)
    print(json.dumps({"checkpoint": a.checkpoint, "samples": val.len(), "accuracy": acc}))


def cmd_predict(a):
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
    sd = load_state_dict(a.input)
    if a.pytorch_keys == "to":
        from ..serialize.state_dict import StateDict
        sd = StateDict.from_tensors(to_pytorch_state_dict(sd))
    elif a.pytorch_keys == "from":
        sd = from_pytorch_state_dict(sd.to_tensors())
    save_state_dict(sd, a.output, Format[a.format] if a.format else detect_format(a.output))
    print(f"{a.input} -> {a.output} ({len(list(sd.keys()))} tensors)")


def cmd_export(a):
    from ..onnx.export import export_module, export_onnx
    cfg, model = _load_model_for(a) if a.checkpoint else (_apply_overrides(ProjectConfig.resolve(a.config), a), None)
    if model is None:
        model = build_model(cfg)
    shape = [1] + [int(s) for s in cfg.model.input_size]
    if cfg.model.architecture.lower() in ("lenet", "simplecnn", "cnn"):
        shape = [1, 1, 28, 28]
    export_onnx(export_module(model, shape, cfg.project.name), a.onnx_path)
    print(f"wrote {a.onnx_path}")


def cmd_inspect(a):
    if a.path.endswith(".gguf"):
        from ..quant.gguf import read_gguf
        g = read_gguf(a.path)
        total = 0
        for name in g.tensor_names():
            info = g.tensors[name]
            shape = list(info["shape"]) if isinstance(info, dict) else list(getattr(info, "shape", []))
            n = 1
            for s in shape:
                n *= s
            total += n
            kind = info.get("type") if isinstance(info, dict) else getattr(info, "type", "")
            print(f"{name:60s} {str(shape):24s} {kind}")
        print(f"{total:,} parameters; metadata keys: {len(g.metadata)}")
        return
    from ..serialize import load_checkpoint, load_state_dict
    try:
        ck = load_checkpoint(a.path)
        sd = ck.model_state
        print(f"checkpoint: epoch {ck.epoch()} step {ck.global_step()} version {ck.axonml_version} config {ck.config}")
    except Exception:
        sd = load_state_dict(a.path)
    total = 0
    for k, v in sd.to_tensors().items():
        total += v.numel()
        print(f"{k:60s} {str(tuple(v.shape)):24s} {str(v.dtype).replace('torch.', '')}")
    print(f"{total:,} parameters")


def cmd_quant(a):
    from ..quant.quantize import compute_quantization_error, dequantize_tensor, quantize_tensor
    from ..quant.types import QuantType
    from ..serialize import load_state_dict, save_state_dict
    qt = QuantType.from_str(a.type) if hasattr(QuantType, "from_str") else QuantType[a.type.upper()]
    sd = load_state_dict(a.input)
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
    from .. import benchmark as B
    if a.what == "hardware":
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
    for spec in a.model or []:
        name, path = spec.split("=", 1)
        inf.load(name, path)
    srv = AxonmlHTTPServer(a.host, a.port, inf, engine)
    print(f"serving on http://{a.host}:{a.port} (models: {[s.split('=')[0] for s in a.model or []]}, llm: {bool(engine)})", flush=True)
    srv.serve_forever()


def cmd_hub(a):
    from .. import hub
    if a.action == "list":
        for m in hub.list_all_models():
            print(f"{m.name:28s} {m.architecture:14s} {m.num_parameters:>14,d}  {m.description}")
    elif a.action == "search":
        for m in hub.search_models(a.query or ""):
            print(m.name)
    else:
        m = hub.get_model_info(a.query)
        print(json.dumps({"name": m.name, "architecture": m.architecture, "parameters": m.num_parameters,
                          "size_mb": m.size_mb(), "tasks": m.tasks, "cached": hub.is_cached(m.name)}))


def cmd_launch(a):
    """One process per GPU on this node: ``axonml launch --nproc 8 script.py [args...]``."""
    n = a.nproc or max(torch.cuda.device_count(), 1)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(a.port), a.script] + a.script_args
    raise SystemExit(subprocess.call(cmd))


def cmd_report(a):
    from ..serialize import load_checkpoint
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

    def common(p):
        p.add_argument("--config", default=os.environ.get("AXONML_CONFIG"))
        p.add_argument("--model"); p.add_argument("--data"); p.add_argument("--device")
        p.add_argument("--output"); p.add_argument("--seed", type=int)
        return p

    p = sub.add_parser("new"); p.add_argument("name"); p.set_defaults(fn=cmd_new)
    p = sub.add_parser("init"); p.add_argument("--force", action="store_true"); p.set_defaults(fn=cmd_init)
    for name, fn in (("train", cmd_train), ("resume", cmd_resume)):
        p = common(sub.add_parser(name))
        p.add_argument("--epochs", type=int); p.add_argument("--batch-size", type=int, dest="batch_size")
        p.add_argument("--lr", type=float); p.add_argument("--optimizer")
        if name == "resume":
            p.add_argument("--checkpoint")
        p.set_defaults(fn=fn)
    p = common(sub.add_parser("eval")); p.add_argument("checkpoint"); p.set_defaults(fn=cmd_eval)
    p = common(sub.add_parser("predict")); p.add_argument("checkpoint"); p.add_argument("--index", type=int, default=0)
    p.set_defaults(fn=cmd_predict)
    p = sub.add_parser("convert"); p.add_argument("input"); p.add_argument("output")
    p.add_argument("--format", choices=["Axonml", "Json", "SafeTensors"]); p.add_argument("--pytorch-keys", choices=["to", "from"])
    p.set_defaults(fn=cmd_convert)
    p = common(sub.add_parser("export")); p.add_argument("onnx_path"); p.add_argument("--checkpoint"); p.set_defaults(fn=cmd_export)
    p = sub.add_parser("inspect"); p.add_argument("path"); p.set_defaults(fn=cmd_inspect)
    p = sub.add_parser("quant"); p.add_argument("input"); p.add_argument("output")
    p.add_argument("--type", default="q8_0"); p.add_argument("--fake", action="store_true")
    p.add_argument("--min-numel", type=int, default=1024); p.set_defaults(fn=cmd_quant)
    p = common(sub.add_parser("bench")); p.add_argument("what", choices=["model", "hardware"], nargs="?", default="model")
    p.add_argument("--batch-sizes", type=int, nargs="+", default=[1, 8, 32]); p.add_argument("--iterations", type=int, default=20)
    p.set_defaults(fn=cmd_bench)
    p = sub.add_parser("gpu"); p.set_defaults(fn=cmd_gpu)
    p = sub.add_parser("serve"); p.add_argument("--host", default="127.0.0.1"); p.add_argument("--port", type=int, default=3021)
    p.add_argument("--model", action="append", help="name=path of a StateDict model"); p.add_argument("--gguf")
    p.add_argument("--max-batch", type=int, default=64); p.add_argument("--max-context", type=int, default=1024)
    p.set_defaults(fn=cmd_serve)
    p = sub.add_parser("hub"); p.add_argument("action", choices=["list", "search", "info"]); p.add_argument("query", nargs="?")
    p.set_defaults(fn=cmd_hub)
    p = sub.add_parser("launch"); p.add_argument("--nproc", type=int, default=0); p.add_argument("--port", type=int, default=29500)
    p.add_argument("script"); p.add_argument("script_args", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_launch)
    p = sub.add_parser("report"); p.add_argument("dir"); p.set_defaults(fn=cmd_report)
    from . import services, workspace
    workspace.add_parsers(sub)
    services.add_parsers(sub)
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    a.fn(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
