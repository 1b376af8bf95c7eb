"""Fused compute+collective kernels on 2+ GPUs against NCCL / single-process references.
Each case runs as one child process per GPU; the NVLS (multimem) path and the plain peer
load/store path are both exercised (``AXONML_NVLS=0`` selects the latter)."""
import pytest
import torch

from tests._mp_gpu import run_gpu_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")]

# the largest power of two of GPUs present, up to 8: the same cases run at 2, 4 and 8 ranks
WORLD = max(w for w in (1, 2, 4, 8) if w <= max(1, torch.cuda.device_count()))


def _fused_allreduce(rank, world, be, dtype_name):
    from axonml_b200 import _native
    from axonml_b200.parallel import ProcessGroup
    from axonml_b200.parallel.fused import FusedAllReduce
    dtype = getattr(torch, dtype_name)
    pg = ProcessGroup(be)
    far = FusedAllReduce.try_create(pg, 3_000_000, dtype)
    assert far is not None
    out = {}
    for n in (1000, 65536 + 24, 2_500_000):
        torch.manual_seed(100 + rank)
        x = torch.randn(n, device="cuda").to(dtype)
        ref = x.clone().float()
        torch.distributed.all_reduce(ref)
        ref = ref / world * 0.5
        inv = torch.tensor([0.5], device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        far.all_reduce_mean_(x, inv_scale=inv, found_inf=flag)
        torch.cuda.synchronize()
        _native.check_status()
        out[n] = ((x.float() - ref).abs().max().item(), int(flag.item()))
    # overflow on one rank only must raise the flag on every rank
    x = torch.ones(4096, device="cuda").to(dtype)
    if rank == world - 1:
        x[4000] = float("inf")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    far.all_reduce_mean_(x, found_inf=flag)
    torch.cuda.synchronize()
    out["inf"] = int(flag.item())
    out["mc"] = bool(far.stage.mc_ptr)
    return out


@pytest.mark.parametrize("nvls", ["1", "0"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_fused_allreduce(dtype, nvls):
    res = run_gpu_ranks(_fused_allreduce, WORLD, args=(dtype,), env={"AXONML_NVLS": nvls})
    tol = 2e-2 if dtype == "bfloat16" else 1e-5
    for r in range(WORLD):
        out = res[r][1]
        for n in (1000, 65536 + 24, 2_500_000):
            err, flag = out[n]
            assert err < tol and flag == 0, (n, err, flag)
        assert out["inf"] == 1


def _oneshot_sum(rank, world, be):
    """The one-trip sum of decode-sized vectors against NCCL, several calls in a row (the two staging
    areas alternate), eager and replayed from a CUDA graph."""
    from axonml_b200 import _native
    from axonml_b200.parallel import ProcessGroup
    from axonml_b200.parallel.fused import FusedAllReduce
    pg = ProcessGroup(be)
    out = {}
    for dtype_name in ("bfloat16", "float32"):
        dtype = getattr(torch, dtype_name)
        far = FusedAllReduce.try_create(pg, 65536, dtype, device_epoch=True)
        assert far is not None
        worst = 0.0
        for it, n in enumerate((4096, 8, 32768 if dtype == torch.bfloat16 else 16384, 4096, 520)):
            torch.manual_seed(7 * it + rank)
            x = torch.randn(n, device="cuda").to(dtype)
            ref = x.clone().float()
            torch.distributed.all_reduce(ref)
            assert far.sum_small_(x, 0.5)
            worst = max(worst, ((x.float() - 0.5 * ref).abs().max() / ref.abs().max()).item())
        # captured once, replayed three times on fresh data
        x = torch.zeros(4096, device="cuda", dtype=dtype)
        src = torch.randn(3, 4096, device="cuda").to(dtype) + rank
        g = torch.cuda.CUDAGraph()
        x.copy_(src[0])
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            far.sum_small_(x)
        for i in range(3):
            x.copy_(src[i])
            g.replay()
            ref = src[i].clone().float()
            torch.distributed.all_reduce(ref)
            worst = max(worst, ((x.float() - ref).abs().max() / ref.abs().max()).item())
        assert not far.sum_small_(torch.zeros(7, device="cuda", dtype=dtype))      # not a multiple of 16 bytes
        torch.cuda.synchronize()
        _native.check_status()
        out[dtype_name] = worst
    return out


@pytest.mark.parametrize("nvls", ["1", "0"])
def test_one_trip_sum_of_small_vectors(nvls):
    res = run_gpu_ranks(_oneshot_sum, WORLD, env={"AXONML_NVLS": nvls})
    for r in range(WORLD):
        assert res[r][1]["bfloat16"] < 2e-2 and res[r][1]["float32"] < 1e-5, res[r][1]


def _arena_heap(rank, world, be):
    """The symmetric heap in arena mode: one exchange, sub-buffers at equal offsets on every rank,
    used by the all-reduce kernels exactly like individually exchanged buffers."""
    from axonml_b200 import _native
    from axonml_b200.parallel import ProcessGroup
    from axonml_b200.parallel.fused import FusedAllReduce
    from axonml_b200.parallel.symm import SymmetricHeap, SymmetricSlice
    pg = ProcessGroup(be)
    heap = SymmetricHeap(pg, arena_bytes=64 << 20)
    far = FusedAllReduce(heap, 1 << 20, torch.bfloat16, device_epoch=True)
    assert isinstance(far.stage, SymmetricSlice) and isinstance(far.comm.signals, SymmetricSlice)
    offs = torch.tensor([far.stage.offset, far.comm.signals.offset, far._small.offset], device="cuda")
    same = [torch.zeros_like(offs) for _ in range(world)]
    torch.distributed.all_gather(same, offs)
    assert all(torch.equal(t, offs) for t in same)                    # equal offsets on every rank
    errs = []
    for n in (4096, 300000):
        torch.manual_seed(3 + rank)
        x = torch.randn(n, device="cuda").bfloat16()
        ref = x.clone().float()
        torch.distributed.all_reduce(ref)
        y = x.clone()
        far.all_reduce_mean_(y)
        errs.append(((y.float() - ref / world).abs().max() / ref.abs().max()).item())
        if n * 2 <= far.SMALL_BYTES:
            z = x.clone()
            assert far.sum_small_(z)
            errs.append(((z.float() - ref).abs().max() / ref.abs().max()).item())
    before = heap.arena_stats()["in_use"]
    tmp = heap.allocate(1000, torch.float32)
    tmp.free()
    assert heap.arena_stats()["in_use"] == before
    big = heap.allocate(80 << 20, torch.uint8)                        # does not fit: its own allocation
    assert not isinstance(big, SymmetricSlice)
    torch.cuda.synchronize()
    _native.check_status()
    return max(errs)


def test_symmetric_heap_arena_mode():
    res = run_gpu_ranks(_arena_heap, WORLD, env={"AXONML_NVLS": "1"})
    for r in range(WORLD):
        assert res[r][1] < 2e-2, res[r][1]


def _fsdp_fused_vs_nccl(rank, world, be):
    import copy
    from axonml_b200 import _native, optim
    from axonml_b200.llm import GPT2Config, GPT2LMHead
    from axonml_b200.parallel import FSDP, ProcessGroup
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=512, n_ctx=128, n_embd=256, n_layer=4, n_head=2, dropout=0.0,
                     attn_dropout=0.0, resid_dropout=0.0)
    base = GPT2LMHead(cfg, device="cuda", dtype=torch.bfloat16)
    m1, m2 = copy.deepcopy(base), copy.deepcopy(base)
    pg = ProcessGroup(be)
    hp = dict(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    f1 = FSDP(m1, pg)
    o1 = optim.AdamW(f1.parameters(), hp["lr"], betas=hp["betas"], eps=hp["eps"], weight_decay=hp["weight_decay"])
    f2 = FSDP(m2, pg, fused_adamw=hp)
    assert f2._fused is not None
    o2 = f2.fused_optimizer()
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (3, 2 * world, 128), generator=g).cuda()
    l1s, l2s = [], []
    for it in range(3):
        x = ids[it].chunk(world)[rank]
        for f, o, ls in ((f1, o1, l1s), (f2, o2, l2s)):
            loss, _ = f.call("forward_with_loss", x)
            loss.backward()
            o.step()
            f.zero_grad()
            ls.append(loss.item())
    torch.cuda.synchronize()
    _native.check_status()
    sd1, sd2 = f1.full_state_dict(), f2.full_state_dict()
    # Adam moves every element by about lr per step, so single elements whose tiny gradients round
    # differently (bf16 NCCL reduction vs fp32 in-kernel reduction) may differ by a few lr; the
    # mean difference must stay far below that.
    diff = max((sd1[k] - sd2[k]).abs().max().item() for k in sd1)
    # global mean: the key-bias third of c_attn.bias has a mathematically zero gradient (softmax is
    # shift invariant), so Adam turns pure rounding noise into +-lr steps there on both paths
    mean = sum((sd1[k] - sd2[k]).abs().sum().item() for k in sd1) / sum(v.numel() for v in sd1.values())
    return l1s, l2s, diff, mean


@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fsdp_fused_rs_adamw_matches_nccl_path(nvls):
    res = run_gpu_ranks(_fsdp_fused_vs_nccl, WORLD, env={"AXONML_NVLS": nvls})
    for r in range(WORLD):
        l1, l2, diff, mean = res[r][1]
        assert abs(l1[-1] - l2[-1]) < 5e-2, (l1, l2)
        assert diff < 1e-2 and mean < 5e-4, (diff, mean)


def _fsdp_fused_gather(rank, world, be):
    """The same model trained with the unit gathers as NCCL all-gathers and with the gathers inside
    the units' first GEMM (activation checkpointing on, so every unit is gathered twice per step)."""
    import copy
    from axonml_b200 import _native, optim
    from axonml_b200.llm import GPT2Config, GPT2LMHead
    from axonml_b200.parallel import FSDP, ProcessGroup
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=512, n_ctx=128, n_embd=256, n_layer=5, n_head=2, dropout=0.0,
                     attn_dropout=0.0, resid_dropout=0.0)
    base = GPT2LMHead(cfg, device="cuda", dtype=torch.bfloat16)
    pg = ProcessGroup(be)
    runs = {}
    for mode in ("nccl", "fused"):
        m = copy.deepcopy(base)
        m.gradient_checkpointing_enable(True)
        m.train()
        f = FSDP(m, pg, gather=mode)
        assert f._k4 == (mode == "fused")
        o = optim.AdamW(f.parameters(), 1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        g = torch.Generator().manual_seed(5)
        ids = torch.randint(0, 512, (3, 2 * world, 128), generator=g).cuda()
        losses = []
        for it in range(3):
            loss, _ = f.call("forward_with_loss", ids[it].chunk(world)[rank])
            loss.backward()
            o.step()
            f.zero_grad()
            losses.append(loss.item())
        torch.cuda.synchronize()
        _native.check_status()
        runs[mode] = (losses, f.full_state_dict(), f.fused_gathers)
    (l1, sd1, n1), (l2, sd2, n2) = runs["nccl"], runs["fused"]
    mean = sum((sd1[k] - sd2[k]).abs().sum().item() for k in sd1) / sum(v.numel() for v in sd1.values())
    return l1, l2, mean, n1, n2


@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fsdp_gather_inside_the_first_gemm_matches_nccl_gathers(nvls):
    res = run_gpu_ranks(_fsdp_fused_gather, WORLD, env={"AXONML_NVLS": nvls})
    for r in range(WORLD):
        l1, l2, mean, n1, n2 = res[r][1]
        # per step: the forward of 5 units, and the recomputation of the 2 units whose rotating buffer
        # was taken over by a later unit (the last 3 are still resident when backward reaches them)
        assert n1 == 0 and n2 == 3 * (5 + 2), (n1, n2)
        assert max(abs(a - b) for a, b in zip(l1, l2)) < 3e-2, (l1, l2)
        assert mean < 5e-4, mean           # three AdamW steps of lr 1e-3 on bf16 gradients summed in another order


def _fsdp_lamb(rank, world, be):
    from axonml_b200 import _native, nn, optim
    from axonml_b200.parallel import FSDP, ProcessGroup
    torch.manual_seed(0)
    mk = lambda: nn.Sequential(nn.Linear(96, 250), nn.Tanh(), nn.Linear(250, 130), nn.Tanh(), nn.Linear(130, 9))
    m = mk().cuda()
    ref = mk().cuda()
    ref.load_state_dict(m.state_dict())
    f = FSDP(m, ProcessGroup(be), param_dtype=torch.float32)
    opt = optim.LAMB(f.parameters(), 2e-2, weight_decay=0.05)
    ropt = optim.LAMB(list(ref.parameters()), 2e-2, weight_decay=0.05)
    g = torch.Generator().manual_seed(5)
    X, Y = torch.randn(3, 8 * world, 96, generator=g).cuda(), torch.randint(0, 9, (3, 8 * world), generator=g).cuda()
    for it in range(3):
        nn.CrossEntropyLoss()(f(X[it].chunk(world)[rank]), Y[it].chunk(world)[rank]).backward()
        opt.step()
        f.zero_grad()
        # the reference sees the same per-rank batches (same kernels, same rounding): LAMB's first
        # steps move every element by about lr * sign(g), so a gradient that is zero up to rounding
        # must round the same way on both sides
        for xs, ys in zip(X[it].chunk(world), Y[it].chunk(world)):
            (nn.CrossEntropyLoss()(ref(xs), ys) / world).backward()
        ropt.step()
        ropt.zero_grad()
    torch.cuda.synchronize()
    _native.check_status()
    sd = f.full_state_dict()
    diffs = [(sd[k] - v.detach()).abs() for k, v in ref.named_parameters()]
    return sum(d.sum().item() for d in diffs) / sum(d.numel() for d in diffs), max(d.max().item() for d in diffs)


def test_fsdp_lamb_trust_ratio_per_tensor_across_shards():
    """The multi-tensor LAMB kernels run on the slices of each tensor that a rank holds; the
    per-tensor sums of squares are all-reduced between the two phases, so sharded LAMB equals
    LAMB on the whole model."""
    res = run_gpu_ranks(_fsdp_lamb, WORLD, env={"AXONML_NVLS": "0"})
    for r in range(WORLD):
        mean, worst = res[r][1]
        # a ratio taken per shard would move whole tensors by ~1e-3; single elements may still
        # differ by 2 * lr * trust where a gradient's sign is decided by the reduction order
        assert mean < 2e-5 and worst < 5e-2, (mean, worst)


def _fsdp_fused_lamb(rank, world, be):
    """LAMB with its first phase inside the reduce-scatter kernel against LAMB stepped on the
    shards after an NCCL reduce-scatter (both take trust ratios per tensor across the shards)."""
    import copy
    from axonml_b200 import _native, optim
    from axonml_b200.llm import GPT2Config, GPT2LMHead
    from axonml_b200.parallel import FSDP, ProcessGroup
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=512, n_ctx=128, n_embd=256, n_layer=4, n_head=2, dropout=0.0,
                     attn_dropout=0.0, resid_dropout=0.0)
    base = GPT2LMHead(cfg, device="cuda", dtype=torch.bfloat16)
    m1, m2 = copy.deepcopy(base), copy.deepcopy(base)
    pg = ProcessGroup(be)
    hp = dict(lr=2e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01)
    f1 = FSDP(m1, pg)
    o1 = optim.LAMB(f1.parameters(), hp["lr"], betas=hp["betas"], eps=hp["eps"], weight_decay=hp["weight_decay"])
    f2 = FSDP(m2, pg, fused_lamb=hp)
    assert f2._fused is not None and f2._fused_kind == "lamb"
    o2 = f2.fused_optimizer()
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (3, 2 * world, 128), generator=g).cuda()
    l1s, l2s = [], []
    for it in range(3):
        x = ids[it].chunk(world)[rank]
        for f, o, ls in ((f1, o1, l1s), (f2, o2, l2s)):
            loss, _ = f.call("forward_with_loss", x)
            loss.backward()
            o.step()
            f.zero_grad()
            ls.append(loss.item())
    torch.cuda.synchronize()
    _native.check_status()
    sd1, sd2 = f1.full_state_dict(), f2.full_state_dict()
    mean = sum((sd1[k] - sd2[k]).abs().sum().item() for k in sd1) / sum(v.numel() for v in sd1.values())
    moved = sum((sd1[k] - base.state_dict()[k].float()).abs().sum().item() for k in sd1) / sum(v.numel() for v in sd1.values())
    return l1s, l2s, mean, moved


@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fsdp_lamb_first_phase_inside_the_reduce_scatter_kernel(nvls):
    res = run_gpu_ranks(_fsdp_fused_lamb, WORLD, env={"AXONML_NVLS": nvls})
    for r in range(WORLD):
        l1, l2, mean, moved = res[r][1]
        assert max(abs(a - b) for a, b in zip(l1, l2)) < 5e-2, (l1, l2)
        # the two runs differ by far less than the three steps moved the parameters
        assert moved > 1e-5 and mean < 0.2 * moved, (mean, moved)


def _ulysses_gpu(rank, world, be):
    from axonml_b200 import _native
    from axonml_b200.ops.attention import sdpa_reference
    from axonml_b200.parallel import ProcessGroup, shard_sequence, ulysses_attention
    pg = ProcessGroup(be)
    g = torch.Generator().manual_seed(11)
    S, Hq, Hkv, D = 256 * world, 2 * world, world, 128
    q = torch.randn(1, S, Hq, D, generator=g).cuda().bfloat16()
    k = torch.randn(1, S, Hkv, D, generator=g).cuda().bfloat16()
    v = torch.randn(1, S, Hkv, D, generator=g).cuda().bfloat16()
    wgt = torch.randn(1, S, Hq, D, generator=g).cuda().bfloat16()
    ql, kl, vl = (shard_sequence(t, pg).clone().requires_grad_(True) for t in (q, k, v))
    o = ulysses_attention(ql, kl, vl, pg, causal=True)
    (o.float() * shard_sequence(wgt, pg).float()).sum().backward()
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    of = sdpa_reference(qf, kf, vf, causal=True)
    (of * wgt.float()).sum().backward()
    torch.cuda.synchronize()
    _native.check_status()
    errs = [(o.float() - shard_sequence(of.detach(), pg)).abs().max().item()]
    for a, full in ((ql.grad, qf.grad), (kl.grad, kf.grad), (vl.grad, vf.grad)):
        ref = shard_sequence(full, pg)
        errs.append(((a.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item())
    return errs


def test_ulysses_context_parallel_attention_on_the_flash_kernels():
    """Sequence-sharded attention: NCCL all-to-all to head shards, the flash-attention kernels on
    the whole sequence, all-to-all back; forward and backward against fp32 attention."""
    res = run_gpu_ranks(_ulysses_gpu, WORLD, env={"AXONML_NVLS": "0"})
    for r in range(WORLD):
        e = res[r][1]
        assert e[0] < 3e-2 and max(e[1:]) < 4e-2, e


def _ddp_fused(rank, world, be):
    from axonml_b200 import nn, optim
    from axonml_b200.parallel import DDP, ProcessGroup
    from axonml_b200.vision import LeNet
    torch.manual_seed(0)
    model = LeNet.new().cuda()
    ddp = DDP(model, ProcessGroup(be), bucket_bytes=64 * 1024)
    fused = bool(ddp._fused)
    opt = optim.SGD(model.parameters(), 0.01).momentum(0.9)
    scaler = optim.GradScaler.with_scale(1024.0)
    ddp.attach_scaler(scaler)
    g = torch.Generator().manual_seed(7)
    X = torch.randn(4, 64, 1, 28, 28, generator=g).cuda()
    Y = torch.randint(0, 10, (4, 64), generator=g).cuda()
    for it in range(4):
        xs, ys = X[it].chunk(world)[rank], Y[it].chunk(world)[rank]
        opt.zero_grad()
        loss = nn.CrossEntropyLoss()(ddp(xs), ys)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
    in_place = all(far.stage.local.data_ptr() <= b.flat.data_ptr() < far.stage.local.data_ptr() + far.capacity * b.flat.element_size()
                   for b in ddp._buckets for far in [ddp._fused.get(b.flat.dtype)] if far is not None)
    return [p.detach().float().cpu() for p in model.parameters()], fused and in_place


def _ddp_mixed_dtypes(rank, world, be):
    """fp32 and bf16 parameters in one model: every dtype gets its own symmetric arena, and the
    result equals the run whose buckets go through the process group."""
    from axonml_b200 import _native, nn, optim
    from axonml_b200.parallel import DDP, ProcessGroup
    outs = []
    for fused in (None, False):
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 16)).cuda()
        model[2].to(torch.bfloat16)
        ddp = DDP(model, ProcessGroup(be), bucket_bytes=4 * 1024, fused=fused)
        if fused is None:
            assert set(ddp._fused) == {torch.float32, torch.bfloat16}
        opt = optim.SGD(model.parameters(), 0.05)
        g = torch.Generator().manual_seed(3)
        X = torch.randn(3, 8 * world, 32, generator=g).cuda()
        for it in range(3):
            opt.zero_grad()
            h = model[1](model[0](X[it].chunk(world)[rank]))
            model[2](h.bfloat16()).float().pow(2).mean().backward()
            opt.step()
        torch.cuda.synchronize()
        _native.check_status()
        outs.append([p.detach().float().cpu() for p in model.parameters()])
    return [(a - b).abs().max().item() for a, b in zip(*outs)]


def test_ddp_fused_allreduce_with_mixed_parameter_dtypes():
    res = run_gpu_ranks(_ddp_mixed_dtypes, WORLD)
    for r in range(WORLD):
        assert max(res[r][1]) < 2e-2, res[r][1]


def test_ddp_fused_allreduce_with_scaler_matches_single_process():
    from axonml_b200 import nn, optim
    from axonml_b200.vision import LeNet
    res = run_gpu_ranks(_ddp_fused, WORLD)
    assert res[0][1][1], "fused all-reduce was not used"
    torch.manual_seed(0)
    ref = LeNet.new()
    opt = optim.SGD(ref.parameters(), 0.01).momentum(0.9)
    g = torch.Generator().manual_seed(7)
    X = torch.randn(4, 64, 1, 28, 28, generator=g)
    Y = torch.randint(0, 10, (4, 64), generator=g)
    for it in range(4):
        opt.zero_grad()
        nn.CrossEntropyLoss()(ref(X[it]), Y[it]).backward()
        opt.step()
    for a, c in zip(res[0][1][0], ref.parameters()):
        assert torch.allclose(a, c.detach(), atol=2e-3), (a - c).abs().max()


def _gemm_comm(rank, world, be):
    """all-gather->GEMM and GEMM->reduce-scatter in one launch each, against NCCL + torch matmul."""
    from axonml_b200 import _native
    from axonml_b200.parallel import ProcessGroup
    from axonml_b200.parallel.gemm_comm import FusedGemmComm
    pg = ProcessGroup(be)
    eng = FusedGemmComm.try_create(pg)
    assert eng is not None
    out = {"mc": bool(eng.ag.sig.mc_ptr)}
    # (Tl, K, N) per call; repeated calls on one engine exercise the epoch / end-of-call protocol
    for i, (tl, k, n) in enumerate([(256, 512, 768), (128, 1024, 256), (512, 2048, 1792), (256, 512, 768)]):
        torch.manual_seed(7 + i)
        w_full = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        torch.manual_seed(100 * i + rank)
        x_local = torch.randn(tl, k, device="cuda").bfloat16()
        bias = torch.randn(n, device="cuda")
        y = eng.ag_gemm(x_local, w_full, bias, "gelu")
        xs = torch.empty(world, tl, k, device="cuda", dtype=torch.bfloat16)
        torch.distributed.all_gather_into_tensor(xs, x_local)
        ref = torch.nn.functional.gelu(xs.view(-1, k).float() @ w_full.float().t() + bias, approximate="tanh")
        torch.cuda.synchronize()
        _native.check_status()
        out[f"ag{i}"] = ((y.float() - ref).abs().max().item(), ref.abs().max().item())
        # row-parallel: every rank multiplies its K slice, rows are scattered
        torch.manual_seed(200 * i + rank)
        x = torch.randn(world * tl, k, device="cuda").bfloat16()
        w_r = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        z = eng.gemm_rs(x, w_r)
        part = x.float() @ w_r.float().t()
        torch.distributed.all_reduce(part)
        ref2 = part[rank * tl:(rank + 1) * tl]
        torch.cuda.synchronize()
        _native.check_status()
        out[f"rs{i}"] = ((z.float() - ref2).abs().max().item(), ref2.abs().max().item())
        # the input-gradient forms: weight read as [K, N]; bias and activation in the reducer
        if k % 128 == 0:
            w_t = w_r.t().contiguous()                               # [k, n]
            z2 = eng.gemm_rs(x, w_t, bias, "relu", trans_b=False)
            ref3 = torch.relu(ref2 + bias)
            y2 = eng.ag_gemm(x_local, w_full.t().contiguous(), trans_b=False, channel=eng.ag_bwd)
            ref4 = xs.view(-1, k).float() @ w_full.float().t()
            torch.cuda.synchronize()
            _native.check_status()
            out[f"rs_t{i}"] = ((z2.float() - ref3).abs().max().item(), ref3.abs().max().item())
            out[f"ag_t{i}"] = ((y2.float() - ref4).abs().max().item(), ref4.abs().max().item())
            # the launch left every rank's rows, its own included, in the kept buffer
            kept = eng.ag_bwd.gathered(world * tl, k)
            out[f"kept{i}"] = ((kept.float() - xs.view(-1, k).float()).abs().max().item(), 0.0)
    return out


@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fused_gemm_allgather_and_reduce_scatter(nvls):
    res = run_gpu_ranks(_gemm_comm, WORLD, env={"AXONML_NVLS": nvls})
    for r in range(WORLD):
        out = res[r][1]
        for key, val in out.items():
            if key == "mc":
                continue
            err, scale = val
            assert err < 0.02 * max(scale, 1.0) + 0.05, (key, err, scale)


def _tp_block_sp(rank, world, be):
    """Sequence-parallel MLP block (column -> swiglu -> row) trained for a few steps through the
    fused kernels must match the same block on the composed NCCL path."""
    from axonml_b200 import _native
    from axonml_b200.parallel import ProcessGroup, fused_gemm
    from axonml_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
    from axonml_b200.ops.elementwise import swiglu
    pg = ProcessGroup(be)
    H, F, tl = 512, 1024, 256
    outs = []
    for fused in (True, False):
        fused_gemm._ENGINES.clear()
        if not fused:
            fused_gemm._ENGINES[id(pg.backend())] = None
        torch.manual_seed(3)
        col = ColumnParallelLinear(H, 2 * F, bias=False, process_group=pg, sequence_parallel=True, device="cuda", dtype=torch.bfloat16)
        row = RowParallelLinear(F, H, bias=False, process_group=pg, sequence_parallel=True, device="cuda", dtype=torch.bfloat16)
        torch.manual_seed(50 + rank)
        x = torch.randn(tl, H, device="cuda").bfloat16().requires_grad_(True)
        y = row(swiglu(col(x)))
        y.float().pow(2).mean().backward()
        torch.cuda.synchronize()
        _native.check_status()
        outs.append((y.detach().float(), x.grad.float(), col.weight.grad.float(), row.weight.grad.float()))
    return [(a - b).abs().max().item() / (b.abs().max().item() + 1e-6) for a, b in zip(*outs)]


def test_sequence_parallel_block_fused_matches_composed():
    res = run_gpu_ranks(_tp_block_sp, WORLD, env={"AXONML_NVLS": "0"})
    for r in range(WORLD):
        for rel in res[r][1]:
            assert rel < 3e-2, res[r][1]


def _vocab_parallel_gpu(rank, world, be):
    """Vocabulary-parallel embedding, head and loss on GPUs against the unsharded computation."""
    from axonml_b200 import _native
    from axonml_b200.parallel import ProcessGroup
    from axonml_b200.parallel.tensor_parallel import (VocabParallelEmbedding, copy_to_tensor_parallel,
                                                       vocab_parallel_cross_entropy)
    pg = ProcessGroup(be)
    V, Vpad, H, T = 1000, 1024, 256, 512            # the real vocabulary does not fill the padded split
    per = Vpad // world
    torch.manual_seed(11)
    table = (torch.randn(Vpad, H, device="cuda") * 0.05).bfloat16()
    head = (torch.randn(Vpad, H, device="cuda") * 0.05).bfloat16()
    ids = torch.randint(0, V, (T,), device="cuda")
    target = torch.randint(0, V, (T,), device="cuda")
    target[::7] = -100
    emb = VocabParallelEmbedding(Vpad, H, pg, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        emb.weight.copy_(table[rank * per:(rank + 1) * per])
    w_local = head[rank * per:(rank + 1) * per].clone().requires_grad_(True)
    launches = _native.launch_count()
    h = emb(ids)
    # the head is column-parallel: each rank's data gradient is a partial sum, added up in backward
    logits = torch.nn.functional.linear(copy_to_tensor_parallel(h, pg), w_local)
    loss = vocab_parallel_cross_entropy(logits, target, pg, rank * per, -100, V)
    loss.backward()
    used_kernels = _native.launch_count() - launches
    torch.cuda.synchronize()
    _native.check_status()
    # unsharded reference in fp32 on the same bf16 values
    tf = table.float().requires_grad_(True)
    hf = head.float().requires_grad_(True)
    h_ref = torch.nn.functional.embedding(ids, tf).bfloat16().float()
    lg = (h_ref @ hf.t())[:, :V]
    ref = torch.nn.functional.cross_entropy(lg, target, ignore_index=-100)
    ref.backward()
    sl = slice(rank * per, (rank + 1) * per)
    return (abs(loss.item() - ref.item()),
            (h.float() - h_ref).abs().max().item(),
            (w_local.grad.float() - hf.grad[sl]).abs().max().item() / (hf.grad.abs().max().item() + 1e-9),
            (emb.weight.grad.float() - tf.grad[sl]).abs().max().item() / (tf.grad.abs().max().item() + 1e-9),
            used_kernels)


def test_vocab_parallel_embedding_head_and_loss_on_gpus():
    res = run_gpu_ranks(_vocab_parallel_gpu, WORLD, env={"AXONML_NVLS": "0"})
    for r in range(WORLD):
        dl, dh, dw, de, used = res[r][1]
        assert dl < 2e-2 and dh < 1e-6 and dw < 5e-2 and de < 5e-2, res[r][1]
        assert used >= 3            # embedding gather, slice statistics, gradient kernel


def _tp_serving_gpu(rank, world, be):
    """Tensor-parallel quantised LLaMA decode: CUDA-graph steps with the peer-memory all-reduce
    against eager steps, same weights, same prompts."""
    import os
    from axonml_b200 import _native
    from axonml_b200.llm import LLaMAConfig
    from axonml_b200.parallel import ProcessGroup
    from axonml_b200.quant import QuantType
    from axonml_b200.server import LLMEngine, QuantizedLlama
    cfg = LLaMAConfig(vocab_size=4096, hidden_size=1024, intermediate_size=2048, num_hidden_layers=3,
                      num_attention_heads=8, num_key_value_heads=8 if world > 4 else 4, max_position_embeddings=256)
    model = QuantizedLlama.from_random(cfg, ProcessGroup(be), device="cuda", std=0.05, proj_type=QuantType.Q4_K)
    prompts = [[(7 * i + j) % 4000 for j in range(24)] for i in range(5)]
    eng = LLMEngine(model, max_batch=8, max_context=64, page_size=16)
    graphs = eng.use_graphs
    eng.warmup([5])
    a = eng.generate(prompts, 6)
    os.environ["AXONML_DECODE_GRAPHS"] = "0"
    b = LLMEngine(model, max_batch=8, max_context=64, page_size=16).generate(prompts, 6)
    torch.cuda.synchronize()
    _native.check_status()
    return a, b, graphs, bool(model._ar)


def test_tensor_parallel_serving_graph_decode_matches_eager():
    res = run_gpu_ranks(_tp_serving_gpu, WORLD)
    a0, b0, graphs, fused = res[0][1]
    assert graphs and fused
    for r in range(WORLD):
        a, b, _, _ = res[r][1]
        assert a == a0 and b == b0          # all ranks agree
    assert a0 == b0


def _skipped_call(rank, world, be):
    """Rank 1 leaves one all-reduce out (host side: it simply does not launch).  Rank 0's kernel
    gives up its wait after the short budget and reports; the next call, made by both, works:
    signals only ever grow, so a call that timed out does not poison the communicator."""
    from axonml_b200 import _native
    from axonml_b200.parallel import ProcessGroup
    from axonml_b200.parallel.fused import FusedAllReduce
    pg = ProcessGroup(be)
    far = FusedAllReduce.try_create(pg, 1 << 16, torch.float32)
    assert far is not None
    x = torch.full((4096,), float(rank + 1), device="cuda")
    far.all_reduce_mean_(x)
    torch.cuda.synchronize()
    _native.check_status()
    out = {"first": x[0].item()}
    _native.set_wait_budget_us(20000)
    y = torch.full((4096,), 5.0, device="cuda")
    if rank == 1:
        far.comm.next_epoch()                     # the call this rank skips
        out["timeout"] = None
    else:
        far.all_reduce_mean_(y)
        torch.cuda.synchronize()
        try:
            _native.check_status()
            out["timeout"] = None
        except _native.KernelTimeout as e:
            out["timeout"] = (e.code, e.where)
    _native.set_wait_budget_us(0)
    torch.cuda.synchronize()
    torch.distributed.barrier()
    z = torch.full((4096,), float(10 * (rank + 1)), device="cuda")
    far.all_reduce_mean_(z)
    torch.cuda.synchronize()
    _native.check_status()
    out["after"] = z[0].item()
    return out


def test_a_skipped_call_times_out_on_the_other_rank_and_the_next_call_works():
    res = run_gpu_ranks(_skipped_call, 2, env={"AXONML_NVLS": "0", "NCCL_NVLS_ENABLE": "0"})
    assert res[0][1]["first"] == res[1][1]["first"] == 1.5
    assert res[0][1]["timeout"] is not None and res[0][1]["timeout"][0] == 3
    assert res[0][1]["after"] == res[1][1]["after"] == 15.0
