"""Headline benchmark: training tokens/s of the GPT-style 1.3B decoder under FSDP ZeRO-3.

Configuration (fixed by the benchmark definition): 24 layers, d_model 2048, 16 heads of 128,
FFN 8192 GELU, pre-LayerNorm, learned positions, vocab 50257; seq 2048, micro-batch 4 per GPU
(weak scaling), AdamW lr 3e-4 betas (0.9, 0.95) wd 0.1, gradient checkpointing on, bf16 compute
with fp32 master weights and optimizer state.  Data: uniform random token ids; weights random-init.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events, max over ranks) with the
inputs already on the device; ``e2e`` is the same loop through the public API with each step's
token ids copied from pinned host memory and the loss read back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="axonml_b200", choices=["axonml_b200", "reference"])
    ap.add_argument("--config", default="gpt1p3b_fsdp")
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count")
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "fused"],
                    help="gradient path at N>1: NCCL reduce-scatter + optimizer, or the fused kernel")
    ap.add_argument("--pp-chunks", type=int, default=1,
                    help="llama8b_tp_pp: model chunks per pipeline rank (> 1 = interleaved 1F1B, reports the transfer/compute split)")
    ap.add_argument("--no-baseline", action="store_true",
                    help="at N>1 skip the second measurement of the same config on plain NCCL collectives")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """The reference is a Rust cargo workspace.  At run time this looks for what its build needs: a
    ``cargo`` on PATH and vendored crates for ``--offline`` (the workspace lists 60+ external crates
    and the machine has no network).  With both present it builds the workspace's CUDA feature set
    and reports that the reference has no entry point for this metric (no multi-GPU transport, no
    LLM trainer binary); without them it prints what it observed."""
    import shutil
    root = os.environ.get("AXONML_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref_src"))
    cargo, rustc = shutil.which("cargo"), shutil.which("rustc")
    pip_tree = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    seen = [f"cargo={'found at ' + cargo if cargo else 'not on PATH'}", f"rustc={'found' if rustc else 'not on PATH'}",
            f"workspace source (AXONML_REFERENCE_ROOT)={'present' if os.path.exists(os.path.join(root, 'Cargo.toml')) else 'not present'}",
            f"vendored crates={'present' if os.path.isdir(os.path.join(root, 'vendor')) else 'absent'}",
            f"pip-installed tree={'present' if os.path.isdir(pip_tree) and os.listdir(pip_tree) else 'absent (no setup.py/pyproject.toml to install)'}"]
    why = "reference is a Rust cargo workspace and cannot be built here: " + "; ".join(seen)
    if cargo and rustc and os.path.exists(os.path.join(root, "Cargo.toml")):
        r = subprocess.run([cargo, "build", "--release", "--offline", "-p", "axonml", "--features", "cuda"], cwd=root,
                           capture_output=True, text=True, timeout=3000)
        if r.returncode == 0:
            why = ("reference built with cargo --offline, but it has no program for this metric: its distributed crate "
                   "has only an in-process mock transport and it ships no LLM/ResNet training binary")
        else:
            why = "cargo build --release --offline failed: " + (r.stderr.strip().splitlines() or ["no output"])[-1][:200]
    print(json.dumps({"impl": "reference", "unavailable": why}))


def bench_q4k_decode(args):
    """GGUF-style Q4_K serving of the Llama-3-8B architecture: p50 time-to-first-token and decode
    tokens/s at concurrent batch 1/8/32/64 (512-token random prompts, greedy decoding)."""
    import torch
    import torch.distributed as dist
    from axonml_b200 import _native
    from axonml_b200.llm import LLaMAConfig
    from axonml_b200.parallel import NcclBackend, ProcessGroup
    from axonml_b200.server import LLMEngine, QuantizedLlama

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    pg = ProcessGroup(NcclBackend.init(timeout_s=600)) if world > 1 else None
    cfg = LLaMAConfig.llama3_8b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    model = QuantizedLlama.from_random(cfg, pg, device=f"cuda:{local}")
    prompt_len, new_tokens = args.seq_len if args.seq_len != 2048 else 512, max(2, args.steps if args.steps > 8 else 256)
    gen = torch.Generator().manual_seed(7)
    results = {}
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _native.launch_count()
    for conc in (1, 8, 32, 64):
        eng = LLMEngine(model, max_batch=64, max_context=prompt_len + new_tokens + 16, page_size=16)
        prompts = torch.randint(0, cfg.vocab_size, (conc, prompt_len), generator=gen).tolist()
        if conc == 1:      # warm-up pass (kernel attributes, allocator)
            LLMEngine(model, 64, prompt_len + 32, 16).generate(prompts, 4)
        eng.warmup([conc])          # decode-graph capture is server start-up, not request time
        eng.generate(prompts, new_tokens)
        st = eng.stats()
        results[conc] = {"ttft_p50_ms": round(st["ttft_p50_s"] * 1e3, 2), "decode_tok_s": round(st["decode_tokens_per_s"], 1),
                         "decode_ms_per_step": round(st["decode_time_s"] / max(st["decode_steps"], 1) * 1e3, 3)}
    launches = _native.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    torch.cuda.synchronize()
    _native.check_status()
    if rank == 0:
        print(json.dumps({"metric": "Q4_K decode tok/s (Llama-3-8B architecture, GGUF Q4_K weights, Q8_0 embeddings/head)",
                          "value": results[64]["decode_tok_s"], "unit": "tokens/s", "n_gpus": world, "steps": new_tokens,
                          "warmup": 4, "ms_per_step": results[64]["decode_ms_per_step"], "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "q4_k weights, bf16 activations/KV",
                          "data": "synthetic", "impl": "axonml_b200",
                          "config": {"model": f"llama-3-8b arch ({cfg.num_hidden_layers}L)", "parallelism": f"tp{world}",
                                     "prompt_len": prompt_len, "new_tokens": new_tokens, "weight_bytes_per_rank": model.weight_bytes(),
                                     "by_concurrency": results, "timing": "host clock around device synchronisation per scheduler step"},
                          "clocks": clocks, "gpu_launches": launches}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def _dist_setup():
    import torch
    from axonml_b200.parallel import NcclBackend, ProcessGroup
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    pg = ProcessGroup(NcclBackend.init(timeout_s=600)) if world > 1 else ProcessGroup.mock()
    return world, rank, local, dev, pg


def timed_training(args, world, rank, local, dev, step_device, step_e2e):
    """Warm-up, K device-timed steps (CUDA events, max over ranks), then K end-to-end steps timed
    on the host around synchronisations (skipped when ``step_e2e`` is None).  Returns the
    measurements of this run."""
    import torch
    import torch.distributed as dist
    from axonml_b200 import _native

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step_device(i)
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for i in range(args.steps):
        loss = step_device(i)
    e1.record()
    sync_all()
    ms_total = e0.elapsed_time(e1)
    launches = _native.launch_count() - launches0
    last_loss = float(loss.item())
    sync_all()
    t0 = time.perf_counter()
    l_host = None
    for i in range(args.steps if step_e2e is not None else 0):
        l_host = step_e2e(i)
    sync_all()
    e2e_ms = (time.perf_counter() - t0) * 1000.0
    clocks = sampler.stop() if rank == 0 else None
    _native.check_status()
    if world > 1:
        t = torch.tensor([ms_total, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = t.tolist()
    return {"ms_per_step": ms_total / args.steps, "e2e_ms_per_step": e2e_ms / args.steps, "launches": launches,
            "clocks": clocks, "last_loss": last_loss, "e2e_last_loss": l_host}


def _finish(world):
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def bench_gpt_fsdp(args):
    import torch
    from axonml_b200 import optim
    from axonml_b200.llm import GPT2Config, GPT2LMHead
    from axonml_b200.parallel import FSDP

    world, rank, local, dev, pg = _dist_setup()
    cfg = GPT2Config.gpt_1_3b()
    if args.layers:
        cfg.n_layer = args.layers
    cfg.n_ctx = max(cfg.n_ctx, args.seq_len)
    hp = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    B, S = args.micro_batch, args.seq_len
    gen = torch.Generator(device="cpu").manual_seed(99 + rank)
    n_host = max(args.steps, 4)
    host_ids = [torch.randint(0, cfg.vocab_size, (B, S), generator=gen).pin_memory() for _ in range(n_host)]
    dev_ids = [t.to(dev) for t in host_ids[:4]]

    def setup(comm):
        """Model, engine and optimizer for one gradient-communication path; returns the two step
        functions and the name of the path actually taken."""
        torch.manual_seed(1234 + rank)
        model = GPT2LMHead(cfg, device=dev, dtype=torch.bfloat16)
        model.gradient_checkpointing_enable(True)
        model.train()
        use_fused = world > 1 and comm in ("auto", "fused")
        engine = FSDP(model, pg, fused_adamw=hp if use_fused else None)
        if engine._fused is not None:
            opt = engine.fused_optimizer()
            path = "fused reduce-scatter+AdamW kernel (peer memory / NVLS)"
        else:
            opt = optim.AdamW(engine.parameters(), hp["lr"], betas=hp["betas"], eps=hp["eps"],
                              weight_decay=hp["weight_decay"])
            path = "nccl" if world > 1 else "none (1 GPU)"

        def run(ids):
            loss, _ = engine.call("forward_with_loss", ids)
            loss.backward()
            opt.step()
            engine.zero_grad()
            return loss

        def step_device(i):
            return run(dev_ids[i % 4])

        def step_e2e(i):
            ids = host_ids[i % n_host].to(dev, non_blocking=True)       # H2D from pinned memory
            return float(run(ids).item())                                 # D2H of the step's result
        nonlocal param_gather
        param_gather = ("fused into each unit's first GEMM (peer memory)" if engine._k4
                        else ("nccl all-gather, prefetched one unit ahead" if world > 1 else "none (1 GPU)"))
        return step_device, step_e2e, path

    param_gather = ""
    step_device, step_e2e, comm_path = setup(args.comm)
    gather_main = param_gather
    m = timed_training(args, world, rank, local, dev, step_device, step_e2e)
    tokens_per_step = B * S * world
    baseline = None
    if world > 1 and comm_path.startswith("fused") and not args.no_baseline:
        # the same config, steps and process group with the gradient path on plain NCCL collectives
        del step_device, step_e2e
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        sd_b, _, path_b = setup("nccl")
        mb = timed_training(args, world, rank, local, dev, sd_b, None)
        baseline = {"grad_comm": path_b, "value": round(tokens_per_step / (mb["ms_per_step"] / 1000.0), 1),
                    "ms_per_step": round(mb["ms_per_step"], 3)}
    if rank == 0:
        out = {
            "metric": "tokens/s 1.3B-FSDP (GPT 1.3B, FSDP ZeRO-3, training)",
            "value": round(tokens_per_step / (m["ms_per_step"] / 1000.0), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(m["ms_per_step"], 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "axonml_b200",
            "config": {"model": "gpt-1.3b (24L d2048 16h ffn8192 vocab50257)",
                       "global_batch": B * world, "seq_len": S, "parallelism": f"fsdp{world}-zero3",
                       "optimizer": "AdamW lr3e-4 b(0.9,0.95) wd0.1", "grad_checkpointing": True,
                       "layers": cfg.n_layer, "grad_comm": comm_path, "param_gather": gather_main,
                       "l2_policy": "per-step working set (weights+optimizer state > 20 GB) far exceeds the 126 MB L2"},
            "clocks": m["clocks"],
            "e2e": {"value": round(tokens_per_step / (m["e2e_ms_per_step"] / 1000.0), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": round(m["e2e_ms_per_step"], 3)},
            "gpu_launches": m["launches"],
            "final_loss": round(m["last_loss"], 4), "e2e_final_loss": round(m["e2e_last_loss"], 4),
        }
        if baseline is not None:
            out["baseline_nccl"] = baseline
        print(json.dumps(out), flush=True)
    return _finish(world)


def bench_llama_tp(args):
    """Llama-style 8B, tensor parallel over all GPUs of the job (sequence-parallel residual stream,
    fused all-gather->GEMM / GEMM->reduce-scatter kernels), AdamW with fp32 master weights.  One
    optimizer step = 8 sequences of 4096 tokens (strong scaling); a rank group of N GPUs runs them
    as 8/N micro-batches of N sequences, so every rank always holds 4096 tokens of the residual
    stream and the activation memory per GPU does not depend on N."""
    import torch
    from axonml_b200 import optim
    from axonml_b200.llm import LLaMAConfig
    from axonml_b200.llm.llama_tp import TPLLaMAForCausalLM
    from axonml_b200.optim.mixed import MasterParams
    from axonml_b200.parallel import fused_gemm

    world, rank, local, dev, pg = _dist_setup()
    cfg = LLaMAConfig.llama3_8b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    S = args.seq_len if args.seq_len != 2048 else 4096
    global_batch = 8
    micro = min(global_batch, world) if args.micro_batch == 4 else args.micro_batch
    n_micro = global_batch // micro
    if args.comm == "nccl":
        fused_gemm._ENGINES[id(pg.backend())] = None         # composed baseline: NCCL + plain GEMM
    torch.manual_seed(4321 + rank)
    model = TPLLaMAForCausalLM(cfg, pg, device=dev, dtype=torch.bfloat16)
    model.train()
    mp = MasterParams(model.parameters())
    opt = optim.AdamW(mp.parameters(), 3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    gen = torch.Generator(device="cpu").manual_seed(77)       # the same ids on every rank
    n_host = max(args.steps, 2)
    host_ids = [torch.randint(0, cfg.vocab_size, (global_batch, S), generator=gen).pin_memory() for _ in range(n_host)]
    dev_ids = [t.to(dev) for t in host_ids[:2]]

    def run(ids):
        total = None
        for j in range(n_micro):
            loss = model.forward_with_loss(ids[j * micro:(j + 1) * micro]) / n_micro
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        model.sync_replicated_grads()
        mp.attach_grads()
        opt.step()
        mp.zero_grad()
        return total

    def step_device(i):
        return run(dev_ids[i % 2])

    def step_e2e(i):
        return float(run(host_ids[i % n_host].to(dev, non_blocking=True)).item())

    m = timed_training(args, world, rank, local, dev, step_device, step_e2e)
    tokens = global_batch * S
    fused = fused_gemm._ENGINES.get(id(pg.backend())) is not None
    baseline = None
    if world > 1 and fused and not args.no_baseline:
        # the same model, steps and process group with every tensor-parallel collective on NCCL
        # around the plain GEMM (the layers look the engine up on every call)
        fused_gemm._ENGINES[id(pg.backend())] = None
        mb = timed_training(args, world, rank, local, dev, step_device, None)
        baseline = {"tp_collectives": "nccl + GEMM", "value": round(tokens / (mb["ms_per_step"] / 1000.0), 1),
                    "ms_per_step": round(mb["ms_per_step"], 3)}
    if rank == 0:
        print(json.dumps({
            **({"baseline_nccl": baseline} if baseline is not None else {}),
            "metric": "tokens/s 8B-TP8 (Llama-style 8B, tensor parallel, training)",
            "value": round(tokens / (m["ms_per_step"] / 1000.0), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(m["ms_per_step"], 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "axonml_b200",
            "config": {"model": f"llama-8b ({cfg.num_hidden_layers}L d4096 32q/8kv ffn14336 vocab128256)",
                       "global_batch": global_batch, "seq_len": S, "parallelism": f"tp{world} (sequence-parallel)",
                       "micro_batches": n_micro, "optimizer": "AdamW lr3e-4 b(0.9,0.95) wd0.1, fp32 master weights",
                       "tp_collectives": "fused all-gather->GEMM / GEMM->reduce-scatter kernels" if fused else
                                         ("nccl + GEMM" if world > 1 else "none (1 GPU)"),
                       "l2_policy": "per-step working set (>= 14 GB of weights and optimizer state per GPU) exceeds the 126 MB L2"},
            "clocks": m["clocks"],
            "e2e": {"value": round(tokens / (m["e2e_ms_per_step"] / 1000.0), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": global_batch * S * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": round(m["e2e_ms_per_step"], 3)},
            "gpu_launches": m["launches"],
            "final_loss": round(m["last_loss"], 4), "e2e_final_loss": round(m["e2e_last_loss"], 4)}), flush=True)
    return _finish(world)


def bench_resnet_ddp(args):
    """ResNet-18, DDP, bf16 autocast with GradScaler, SGD momentum 0.9, channels-last, batch 256
    per GPU (weak scaling), 25 MB gradient buckets overlapped with backward."""
    import torch
    from axonml_b200 import nn, optim
    from axonml_b200.autograd.amp import autocast
    from axonml_b200.parallel import DDP
    from axonml_b200.vision.models.resnet import resnet18

    world, rank, local, dev, pg = _dist_setup()
    torch.manual_seed(1)
    model = resnet18(1000).to(dev).to(memory_format=torch.channels_last)
    model.train()
    ddp = DDP(model, pg, bucket_bytes=25 * 1024 * 1024)
    opt = optim.SGD(model.parameters(), 0.1).momentum(0.9)
    scaler = optim.GradScaler.new()
    ddp.attach_scaler(scaler)
    crit = nn.CrossEntropyLoss()
    B = 256 if args.micro_batch == 4 else args.micro_batch
    gen = torch.Generator(device="cpu").manual_seed(5 + rank)
    n_host = 3
    host_x = [torch.randn(B, 3, 224, 224, generator=gen).to(torch.bfloat16).contiguous(memory_format=torch.channels_last).pin_memory()
              for _ in range(n_host)]
    host_y = [torch.randint(0, 1000, (B,), generator=gen).pin_memory() for _ in range(n_host)]
    dev_x = [t.to(dev) for t in host_x]
    dev_y = [t.to(dev) for t in host_y]

    def run(x, y):
        opt.zero_grad()
        with autocast(torch.bfloat16):
            loss = crit(ddp(x), y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        return loss.detach()

    def step_device(i):
        return run(dev_x[i % n_host], dev_y[i % n_host])

    def step_e2e(i):
        x = host_x[i % n_host].to(dev, non_blocking=True)
        y = host_y[i % n_host].to(dev, non_blocking=True)
        return float(run(x, y).item())

    m = timed_training(args, world, rank, local, dev, step_device, step_e2e)
    imgs = B * world
    baseline = None
    grad_comm = "fused all-reduce+unscale kernel, buckets reduced in place in symmetric memory" if ddp._fused else ("nccl" if world > 1 else "none (1 GPU)")
    if world > 1 and ddp._fused and not args.no_baseline:
        # the same model, steps and process group with the bucket all-reduce on NCCL
        ddp._fused = {}
        mb = timed_training(args, world, rank, local, dev, step_device, None)
        baseline = {"grad_comm": "nccl", "value": round(imgs / (mb["ms_per_step"] / 1000.0), 1),
                    "ms_per_step": round(mb["ms_per_step"], 3)}
    if rank == 0:
        print(json.dumps({
            **({"baseline_nccl": baseline} if baseline is not None else {}),
            "metric": "ResNet-18 img/s (DDP, bf16 AMP, training)",
            "value": round(imgs / (m["ms_per_step"] / 1000.0), 1), "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(m["ms_per_step"], 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast (fp32 params)",
            "data": "synthetic", "impl": "axonml_b200",
            "config": {"model": "resnet18 (1000 classes)", "global_batch": imgs, "image": "3x224x224 channels-last",
                       "parallelism": f"ddp{world}", "optimizer": "SGD momentum 0.9 + GradScaler",
                       "bucket_mb": 25, "grad_comm": grad_comm,
                       "l2_policy": "per-step activations (> 10 GB) exceed the 126 MB L2"},
            "clocks": m["clocks"],
            "e2e": {"value": round(imgs / (m["e2e_ms_per_step"] / 1000.0), 1), "unit": "images/s",
                    "h2d_bytes_per_step": B * 3 * 224 * 224 * 2 + B * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": round(m["e2e_ms_per_step"], 3)},
            "gpu_launches": m["launches"], "final_loss": round(m["last_loss"], 4)}), flush=True)
    return _finish(world)


def bench_lenet_cpu(args):
    """LeNet-5 fp32 on the CPU, 100 SGD steps of batch 64; with --gpus 2 the same job as two DDP
    ranks over the CPU (gloo) process group.  Needs no GPU."""
    import torch
    from axonml_b200 import nn, optim
    from axonml_b200.parallel import CpuBackend, DDP, ProcessGroup
    from axonml_b200.vision import LeNet

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    pg = ProcessGroup(CpuBackend.init(timeout_s=120)) if world > 1 else ProcessGroup.mock()
    torch.manual_seed(0)
    model = LeNet.new()
    net = DDP(model, pg) if world > 1 else model
    opt = optim.SGD(model.parameters(), 0.01).momentum(0.9)
    crit = nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(42 + rank)
    steps = args.steps if args.steps != 8 else 100
    X = torch.randn(steps, 64, 1, 28, 28, generator=g)
    Y = torch.randint(0, 10, (steps, 64), generator=g)

    def step(i):
        opt.zero_grad()
        loss = crit(net(X[i]), Y[i])
        loss.backward()
        opt.step()
        return float(loss)

    for i in range(min(args.warmup, steps)):
        step(i)
    t0 = time.perf_counter()
    for i in range(steps):
        last = step(i)
    dt = time.perf_counter() - t0
    if rank == 0:
        print(json.dumps({"metric": "LeNet-5 CPU training images/s", "value": round(64 * world * steps / dt, 1),
                          "unit": "images/s", "n_gpus": 0, "steps": steps, "warmup": args.warmup,
                          "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "axonml_b200",
                          "config": {"model": "lenet5", "global_batch": 64 * world, "parallelism": f"cpu-ddp{world}",
                                     "optimizer": "SGD lr0.01 momentum0.9"},
                          "gpu_launches": 0, "final_loss": round(last, 4)}), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return 0


def bench_llama_tp_pp(args):
    """Llama-style 8B as TP = N/2 x PP = 2 (stage s = ranks [s*TP, (s+1)*TP)), 1F1B over 8 microbatches
    of one 4096-token sequence, AdamW with fp32 master weights.  Activations between the stages are
    the sequence-parallel token shards, sent rank-to-rank over NCCL p2p."""
    import torch
    from axonml_b200 import optim
    from axonml_b200.llm import LLaMAConfig
    from axonml_b200.llm.llama_tp import build_tp_pp
    from axonml_b200.optim.mixed import MasterParams
    from axonml_b200.parallel import World, fused_gemm

    world, rank, local, dev, pg = _dist_setup()
    if world < 2 or world % 2:
        raise SystemExit("llama8b_tp_pp needs an even number of GPUs (TP = N/2, PP = 2)")
    cfg = LLaMAConfig.llama3_8b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    S = args.seq_len if args.seq_len != 2048 else 4096
    global_batch, n_micro = 8, 8
    torch.manual_seed(4321 + rank)
    w = World.init(pg.backend())
    pipe, stage, tp_pg = build_tp_pp(cfg, w, world // 2, 2, S, device=dev, dtype=torch.bfloat16, num_microbatches=n_micro,
                                     chunks=args.pp_chunks)
    if args.comm == "nccl":
        fused_gemm._ENGINES[id(tp_pg.backend())] = None
    stage.train()
    mp = MasterParams(stage.parameters())
    opt = optim.AdamW(mp.parameters(), 3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    gen = torch.Generator(device="cpu").manual_seed(77)
    n_host = max(args.steps, 2)
    host_ids = [torch.randint(0, cfg.vocab_size, (global_batch, S), generator=gen).pin_memory() for _ in range(n_host)]
    dev_ids = [t.to(dev) for t in host_ids[:2]]
    last_stage = stage.model.last_stage

    def run(ids):
        loss = pipe.train_step(ids, ids, stage.loss, act_dtype=torch.bfloat16)
        stage.model.sync_replicated_grads()
        mp.attach_grads()
        opt.step()
        mp.zero_grad()
        return loss if loss is not None else torch.zeros((), device=dev)

    def step_device(i):
        return run(dev_ids[i % 2])

    def step_e2e(i):
        return float(run(host_ids[i % n_host].to(dev, non_blocking=True)).item())

    m = timed_training(args, world, rank, local, dev, step_device, step_e2e)
    # the loss lives on the last stage: fetch it for the report
    import torch.distributed as dist
    t = torch.tensor([m["last_loss"] if last_stage else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tokens = global_batch * S
    # interleaved schedule: how long the last step waited for transfers against how long it computed (max over ranks)
    pipeline = None
    if pipe.last_comm is not None:
        c = torch.tensor([pipe.last_comm["wait_s"], pipe.last_comm["compute_s"]], device=dev)
        dist.all_reduce(c, op=dist.ReduceOp.MAX)
        pipeline = {"schedule": f"interleaved 1F1B, {args.pp_chunks} chunks per rank", "wait_ms_max": round(c[0].item() * 1e3, 2),
                    "compute_ms_max": round(c[1].item() * 1e3, 2),
                    "wait_fraction": round(c[0].item() / max(c[0].item() + c[1].item(), 1e-9), 3),
                    "timing": "host clock around the receives and around the stage computations of the last step"}
    if rank == 0:
        print(json.dumps({
            "pipeline": pipeline,
            "metric": "tokens/s 8B TP x PP (Llama-style 8B, tensor + pipeline parallel, training)",
            "value": round(tokens / (m["ms_per_step"] / 1000.0), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(m["ms_per_step"], 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "axonml_b200",
            "config": {"model": f"llama-8b ({cfg.num_hidden_layers}L d4096 32q/8kv ffn14336 vocab128256)",
                       "global_batch": global_batch, "seq_len": S, "parallelism": f"tp{world // 2} x pp2 ({'interleaved ' if args.pp_chunks > 1 else ''}1F1B, {n_micro} microbatches)",
                       "optimizer": "AdamW lr3e-4 b(0.9,0.95) wd0.1, fp32 master weights",
                       "l2_policy": "per-step working set (>= 14 GB per GPU) exceeds the 126 MB L2"},
            "clocks": m["clocks"],
            "e2e": {"value": round(tokens / (m["e2e_ms_per_step"] / 1000.0), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": global_batch * S * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": round(m["e2e_ms_per_step"], 3)},
            "gpu_launches": m["launches"], "final_loss": round(float(t.item()), 4)}), flush=True)
    return _finish(world)


def bench_published_micro(args):
    """The four operations of the reference's published table (docs/index.md:128-133: MatMul
    1024x1024 f32 2.1 ms, Conv2d 224x224 4.3 ms, LSTM seq 128 8.2 ms, Adam step 0.8 ms, one CPU
    thread of a Ryzen 9 5900X) timed here on one CPU thread of this host and, when a GPU is present,
    on this package's kernels.  The table does not state the convolution's channels, the LSTM's
    width or the Adam parameter count; the shapes used are given in `config`."""
    os.environ.setdefault("OMP_NUM_THREADS", "1")       # the published table is single-threaded
    import torch
    from axonml_b200 import nn, optim
    published = {"matmul_1024_f32": 2.1, "conv2d_224": 4.3, "lstm_seq128": 8.2, "adam_step": 0.8}
    iters = args.steps if args.steps != 8 else 20

    def cpu_ms(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        return (time.perf_counter() - t0) / iters * 1e3

    def gpu_ms(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def build(dev, dt):
        torch.manual_seed(0)
        a, b = torch.randn(1024, 1024, device=dev, dtype=dt), torch.randn(1024, 1024, device=dev, dtype=dt)
        conv = nn.Conv2d(3, 16, 3, 1, 1).to(dev, dt)
        x = torch.randn(1, 3, 224, 224, device=dev, dtype=dt)
        if dev == "cuda":
            x = x.contiguous(memory_format=torch.channels_last)
        lstm = nn.LSTM(128, 128, 1).to(dev, dt)
        seq = torch.randn(1, 128, 128, device=dev, dtype=dt)
        lin = nn.Linear(1000, 1000).to(dev)
        opt = optim.Adam(list(lin.parameters()), 1e-3)
        for p in lin.parameters():
            p.grad = torch.randn_like(p)
        with torch.no_grad():
            ops = {"matmul_1024_f32": lambda: a @ b, "conv2d_224": lambda: conv(x), "lstm_seq128": lambda: lstm(seq)}
        ops["adam_step"] = opt.step
        return ops

    torch.set_num_threads(1)
    cpu_ops = build("cpu", torch.float32)
    # CPU column: this repo's own C++ reference kernels where it has one (blocked sgemm, direct
    # convolution: the restatement of the reference's CPU algorithms, on one thread), the
    # package's CPU path (torch operators) for the LSTM and the Adam step
    from axonml_b200.core.backends import CpuBackend
    ca, cb = torch.randn(1024, 1024), torch.randn(1024, 1024)
    cw, cbias, cx = torch.randn(16, 3, 3, 3), torch.randn(16), torch.randn(1, 3, 224, 224)
    cpu_ops["matmul_1024_f32"] = lambda: CpuBackend.matmul(ca, cb)
    cpu_ops["conv2d_224"] = lambda: CpuBackend.conv2d(cx, cw, cbias, 1, 1)
    res = {}
    with torch.no_grad():
        for k in ("matmul_1024_f32", "conv2d_224", "lstm_seq128"):
            res[k] = {"cpu_ms": round(cpu_ms(cpu_ops[k]), 3)}
    res["adam_step"] = {"cpu_ms": round(cpu_ms(cpu_ops["adam_step"]), 3)}
    for k, who in (("matmul_1024_f32", "C++ reference kernel"), ("conv2d_224", "C++ reference kernel"),
                   ("lstm_seq128", "package CPU path (torch operators)"), ("adam_step", "package CPU path (torch operators)")):
        res[k]["cpu_impl"] = who
    launches = 0
    if torch.cuda.is_available():
        from axonml_b200 import _native
        from axonml_b200.ops.gemm import sgemm_f32
        gpu_ops = build("cuda", torch.bfloat16)
        ga, gb = torch.randn(1024, 1024, device="cuda"), torch.randn(1024, 1024, device="cuda")
        n0 = _native.cuda().launches
        with torch.no_grad():
            # the published row is f32: the comparable GPU number is the fp32 GEMM; the bf16
            # tensor-core time is reported beside it and does not enter the mean
            res["matmul_1024_f32"]["gpu_ms"] = round(gpu_ms(lambda: sgemm_f32(ga, gb)), 4)
            res["matmul_1024_f32"]["gpu_bf16_ms_not_comparable"] = round(gpu_ms(gpu_ops["matmul_1024_f32"]), 4)
            for k in ("conv2d_224", "lstm_seq128"):
                res[k]["gpu_ms"] = round(gpu_ms(gpu_ops[k]), 4)
                res[k]["gpu_dtype"] = "bf16 (the published row states no dtype for the GPU; fp32 on the CPU)"
        res["adam_step"]["gpu_ms"] = round(gpu_ms(gpu_ops["adam_step"]), 4)
        launches = _native.cuda().launches - n0
    on_gpu = torch.cuda.is_available()
    geo = 1.0
    for k, v in res.items():
        v["published_ms"] = published[k]
        v["published_over_cpu"] = round(published[k] / v["cpu_ms"], 2)
        if on_gpu:
            v["published_over_gpu"] = round(published[k] / v["gpu_ms"], 1)
        geo *= published[k] / (v["gpu_ms"] if on_gpu else v["cpu_ms"])
    geo **= 0.25
    where = "one B200, this package's kernels" if on_gpu else "1 CPU thread of this host"
    print(json.dumps({"metric": "published CPU micro-table (matmul 1024^2, conv2d 224^2, LSTM seq 128, Adam step)",
                      "value": round(geo, 3), "unit": f"x the published speed (geometric mean of published ms / ours; {where})",
                      "n_gpus": 1 if torch.cuda.is_available() else 0, "steps": iters, "warmup": max(args.warmup, 3),
                      "ms_per_step": None, "higher_is_better": True, "scaling": "strong", "vs_baseline": round(geo, 3),
                      "dtype": "fp32 (matmul and Adam on both devices; convolution and LSTM run bf16 on the GPU)", "data": "synthetic", "impl": "axonml_b200",
                      "config": {"matmul": "1024x1024x1024", "conv2d": "1x3x224x224, 16 filters 3x3 pad 1",
                                 "lstm": "1 layer, 128 -> 128, sequence 128, batch 1", "adam": "1000x1000 weight + bias",
                                 "l2_policy": "operands fit in cache, as in the published table"},
                      "ops": res, "gpu_launches": launches}), flush=True)
    return 0


def main():
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            reference_arm(args)
        return 0
    if args.config == "q4k_decode":
        return bench_q4k_decode(args)
    if args.config == "llama8b_tp":
        return bench_llama_tp(args)
    if args.config == "llama8b_tp_pp":
        return bench_llama_tp_pp(args)
    if args.config == "resnet18_ddp":
        return bench_resnet_ddp(args)
    if args.config == "lenet_cpu":
        return bench_lenet_cpu(args)
    if args.config == "published_micro":
        return bench_published_micro(args)
    return bench_gpt_fsdp(args)


if __name__ == "__main__":
    sys.exit(main())
