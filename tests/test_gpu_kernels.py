"""Numerics of the hand-written sm_100a kernels against plain PyTorch fp32 references.

Mirrors the reference's CPU-vs-GPU harness (crates/axonml-core/src/backends/gpu_tests.rs:221-367):
deterministic inputs, a sweep of sizes that includes ragged tails, absolute + relative tolerance.
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DEV = "cuda"


def close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    assert bool((err <= lim).all()), f"max err {err.max().item():.4g} (limit {lim.max().item():.4g})"


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 264, 136), (1024, 1024, 1024), (8, 8, 8),
                                   (4096, 512, 2048)])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, ta, tb, kernel_status):
    from axonml_b200.ops.gemm import gemm_bf16
    a = torch.randn((K, M) if ta else (M, K), device=DEV).bfloat16()
    b = torch.randn((N, K) if tb else (K, N), device=DEV).bfloat16()
    c = gemm_bf16(a, b, trans_a=ta, trans_b=tb)
    A = a.float().t() if ta else a.float()
    B = b.float().t() if tb else b.float()
    ref = A @ B
    close(c, ref, atol=0.02 * (K ** 0.5), rtol=2e-2)


@pytest.mark.parametrize("act", ["none", "relu", "gelu", "silu", "sigmoid", "tanh"])
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_epilogue(act, bn, kernel_status):
    from axonml_b200.ops.gemm import gemm_bf16
    M, N, K = 384, 512, 256
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).bfloat16()
    bias = torch.randn(N, device=DEV)
    y, z = gemm_bf16(a, w, bias=bias, act=act, want_aux=True, bn=bn)
    zr = a.float() @ w.float().t() + bias
    fn = {"none": lambda t: t, "relu": torch.relu, "gelu": lambda t: F.gelu(t, approximate="tanh"),
          "silu": F.silu, "sigmoid": torch.sigmoid, "tanh": torch.tanh}[act]
    close(z, zr, 2e-2, 2e-2)
    close(y, fn(zr), 2e-2, 2e-2)


@pytest.fixture
def pair_mode():
    from axonml_b200.ops.gemm import set_pair_mode
    set_pair_mode(1)
    yield
    set_pair_mode(-1)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 384, 192), (328, 264, 136), (2048, 1024, 1024),
                                   (4096, 512, 2048), (136, 128, 72), (8192, 640, 520)])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_cta_pair_layouts(M, N, K, ta, tb, bn, pair_mode, kernel_status):
    """The two-CTA kernel (each CTA loads its half of the operands, the even CTA issues M = 256
    MMAs) against an fp32 matmul, ragged edges in every dimension included."""
    from axonml_b200.ops.gemm import gemm_bf16
    a = torch.randn((K, M) if ta else (M, K), device=DEV).bfloat16()
    b = torch.randn((N, K) if tb else (K, N), device=DEV).bfloat16()
    c = gemm_bf16(a, b, trans_a=ta, trans_b=tb, bn=bn)
    A = a.float().t() if ta else a.float()
    B = b.float().t() if tb else b.float()
    close(c, A @ B, atol=0.02 * (K ** 0.5), rtol=2e-2)
    # the one-CTA kernel accumulates in the same order: results agree to the last bf16 bit or so
    from axonml_b200.ops.gemm import set_pair_mode
    set_pair_mode(0)
    c1 = gemm_bf16(a, b, trans_a=ta, trans_b=tb, bn=bn)
    set_pair_mode(1)
    close(c, c1, atol=1e-2 * (K ** 0.5) * 0.1, rtol=1e-2)


@pytest.mark.parametrize("act", ["none", "gelu", "silu"])
@pytest.mark.parametrize("bn", [0, 128, 256])
def test_gemm_cta_pair_epilogue(act, bn, pair_mode, kernel_status):
    from axonml_b200.ops.gemm import gemm_bf16
    M, N, K = 640, 512, 256
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).bfloat16()
    bias = torch.randn(N, device=DEV)
    y, z = gemm_bf16(a, w, bias=bias, act=act, want_aux=True, bn=bn)
    zr = a.float() @ w.float().t() + bias
    fn = {"none": lambda t: t, "gelu": lambda t: F.gelu(t, approximate="tanh"), "silu": F.silu}[act]
    close(z, zr, 2e-2, 2e-2)
    close(y, fn(zr), 2e-2, 2e-2)


def test_gemm_cta_pair_many_waves(pair_mode, kernel_status):
    """More tiles than CTA pairs: the stage ring, both accumulators and the barrier phases wrap
    several times."""
    from axonml_b200.ops.gemm import gemm_bf16
    a = torch.randn(8192, 512, device=DEV).bfloat16()
    b = torch.randn(4096, 512, device=DEV).bfloat16()
    for bn in (128, 256):
        c = gemm_bf16(a, b, bn=bn)
        close(c, a.float() @ b.float().t(), atol=0.02 * 512 ** 0.5, rtol=2e-2)


def test_linear_autograd(kernel_status):
    from axonml_b200.ops.linear import linear
    x = torch.randn(4, 96, 256, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device=DEV) / 16).bfloat16().requires_grad_()
    b = torch.randn(512, device=DEV).bfloat16().requires_grad_()
    y = linear(x, w, b, "gelu")
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.gelu(F.linear(xr, wr, br), approximate="tanh")
    yr.backward(g.float())
    close(y, yr, 3e-2, 3e-2)
    close(x.grad, xr.grad, 5e-2, 5e-2)
    close(w.grad, wr.grad, 0.3, 5e-2)
    close(b.grad, br.grad, 0.3, 5e-2)


# ------------------------------------------------------------------ norms
@pytest.mark.parametrize("rows,D", [(1, 8), (7, 64), (33, 256), (512, 2048), (100, 4096), (64, 1000)])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_fwd_bwd(rows, D, rms, dtype):
    from axonml_b200.ops.norm import layer_norm, rms_norm
    x = torch.randn(rows, D, device=DEV).to(dtype).requires_grad_()
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(dtype).requires_grad_()
    b = (0.1 * torch.randn(D, device=DEV)).to(dtype).requires_grad_()
    y = rms_norm(x, w, 1e-5) if rms else layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        yr = F.layer_norm(xr, (D,), wr, br, 1e-5)
    yr.backward(g.float())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    close(y, yr, tol, tol)
    close(x.grad, xr.grad, tol, tol)
    wt = 1e-3 if dtype == torch.float32 else 0.05 * rows ** 0.5
    close(w.grad, wr.grad, wt, 2e-2)
    if not rms:
        close(b.grad, br.grad, wt, 2e-2)


def test_norm_residual():
    from axonml_b200.ops.norm import layer_norm
    x = torch.randn(64, 512, device=DEV).bfloat16().requires_grad_()
    r = torch.randn(64, 512, device=DEV).bfloat16().requires_grad_()
    w = torch.ones(512, device=DEV).bfloat16().requires_grad_()
    b = torch.zeros(512, device=DEV).bfloat16().requires_grad_()
    y, h = layer_norm(x, w, b, 1e-5, residual=r)
    (y.float().sum() + (h.float() ** 2).sum()).backward()
    xr, rr = x.detach().float().requires_grad_(), r.detach().float().requires_grad_()
    hr = (xr + rr)
    yr = F.layer_norm(hr, (512,))
    (yr.sum() + (hr ** 2).sum()).backward()
    close(h, hr, 2e-2, 2e-2)
    close(y, yr, 3e-2, 3e-2)
    close(x.grad, xr.grad, 0.1, 5e-2)
    close(r.grad, rr.grad, 0.1, 5e-2)


# ------------------------------------------------------------------ softmax / CE
@pytest.mark.parametrize("rows,V", [(1, 1), (7, 10), (16, 1000), (64, 50257), (4, 128256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cross_entropy(rows, V, dtype):
    from axonml_b200.ops.loss import cross_entropy
    Vpad = (V + 127) // 128 * 128
    logits = (3 * torch.randn(rows, Vpad, device=DEV)).to(dtype).requires_grad_()
    t = torch.randint(0, V, (rows,), device=DEV)
    if rows > 4:
        t[1] = -100
    loss = cross_entropy(logits, t, valid_classes=V)
    loss.backward()
    lr = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lr[:, :V], t, ignore_index=-100)
    ref.backward()
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    close(loss, ref, tol, tol)
    close(logits.grad, lr.grad, tol / 10, tol)


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("shape,dim", [((4, 7), -1), ((3, 5, 64), 1), ((16, 4096), -1)])
def test_softmax(shape, dim, log):
    from axonml_b200.ops.loss import softmax
    x = torch.randn(*shape, device=DEV).requires_grad_()
    y = softmax(x, dim, log=log)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().clone().requires_grad_()
    yr = F.log_softmax(xr, dim) if log else F.softmax(xr, dim)
    yr.backward(g)
    close(y, yr, 1e-5, 1e-4)
    close(x.grad, xr.grad, 1e-5, 1e-3)


# ------------------------------------------------------------------ elementwise set
@pytest.mark.parametrize("n", [1, 7, 16, 64, 256, 1024, 4096, 100003])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_elementwise_set(n, dtype):
    from axonml_b200.ops import elementwise as E
    x = torch.randn(n, device=DEV).to(dtype)
    y = torch.randn(n, device=DEV).to(dtype)
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    approx = dict(atol=1e-3, rtol=1e-2) if dtype == torch.float32 else tol
    for op in ("add", "sub", "mul", "max", "min"):
        close(E.binary(x, y, op), E._binary_ref(x.float(), y.float(), op, 0.0), **tol)
    close(E.binary(x, y.abs() + 0.5, "div"), x.float() / (y.float().abs() + 0.5), **approx)
    for op, p0, p1 in (("neg", 0, 0), ("abs", 0, 0), ("relu", 0, 0), ("scale", 2.5, 0),
                       ("add_scalar", -1.25, 0), ("clamp", -0.5, 0.5), ("square", 0, 0),
                       ("leaky_relu", 0.01, 0)):
        close(E.unary(x, op, p0, p1), E._UNARY_REF[op](x.float(), p0, p1), **tol)
    for op, p0 in (("sigmoid", 0), ("tanh", 0), ("gelu", 0), ("silu", 0), ("elu", 1.0), ("exp", 0)):
        close(E.unary(x, op, p0), E._UNARY_REF[op](x.float(), p0, 0), **approx)
    xp = x.abs() + 0.1
    for op in ("sqrt", "log", "rsqrt"):
        close(E.unary(xp, op), E._UNARY_REF[op](xp.float(), 0, 0), **approx)
    for act in ("relu", "gelu", "silu"):
        close(E.act_backward(y, x, act), E._binary_ref(y.float(), x.float(), act + "_bwd", 0.0), **approx)


def test_swiglu_and_colsum():
    from axonml_b200.ops import elementwise as E
    gu = torch.randn(37, 2 * 256, device=DEV).bfloat16().requires_grad_()
    out = E.swiglu(gu)
    g = torch.randn_like(out)
    out.backward(g)
    gr = gu.detach().float().requires_grad_()
    a, b = gr.split(256, -1)
    ref = F.silu(a) * b
    ref.backward(g.float())
    close(out, ref, 2e-2, 2e-2)
    close(gu.grad, gr.grad, 3e-2, 3e-2)
    x = torch.randn(3000, 520, device=DEV).bfloat16()
    close(E.colsum(x), x.float().sum(0), 1e-2, 1e-3)


def test_dropout():
    from axonml_b200.ops import elementwise as E
    x = torch.ones(1 << 20, device=DEV, requires_grad=True)
    y = E.dropout(x, 0.25, True)
    keep = (y != 0).float().mean().item()
    assert abs(keep - 0.75) < 0.01
    assert torch.allclose(y[y != 0], torch.full_like(y[y != 0], 1 / 0.75))
    y.sum().backward()
    assert torch.equal(x.grad != 0, y != 0)


# ------------------------------------------------------------------ embedding / rope
def test_embedding_and_rope():
    from axonml_b200.ops import misc as Mi
    V, D, B, S = 1000, 256, 3, 17
    W = torch.randn(V, D, device=DEV).bfloat16().requires_grad_()
    P = torch.randn(64, D, device=DEV).bfloat16().requires_grad_()
    idx = torch.randint(0, V, (B, S), device=DEV)
    out = Mi.embedding(idx, W, pos_weight=P, seq_len=S)
    g = torch.randn_like(out)
    out.backward(g)
    Wr, Pr = W.detach().float().requires_grad_(), P.detach().float().requires_grad_()
    ref = F.embedding(idx, Wr) + Pr[:S][None]
    ref.backward(g.float())
    close(out, ref, 2e-2, 2e-2)
    close(W.grad, Wr.grad, 5e-2, 2e-2)
    close(P.grad, Pr.grad, 5e-2, 2e-2)

    H, hd = 4, 128
    cos, sin = Mi.rope_tables(64, hd, 500000.0, device=DEV)
    x = torch.randn(B, S, H, hd, device=DEV).bfloat16().requires_grad_()
    y = Mi.rope(x, cos, sin, seq_len=S)
    y.backward(torch.ones_like(y))
    xr = x.detach().float().requires_grad_()
    c, s = cos[:S].view(1, S, 1, hd // 2), sin[:S].view(1, S, 1, hd // 2)
    a, b = xr[..., :hd // 2], xr[..., hd // 2:]
    yr = torch.cat([a * c - b * s, b * c + a * s], -1)
    yr.backward(torch.ones_like(yr))
    close(y, yr, 2e-2, 2e-2)
    close(x.grad, xr.grad, 2e-2, 2e-2)


# ------------------------------------------------------------------ fused optimizers
@pytest.mark.parametrize("kind", ["sgd", "adam", "adamw", "rmsprop", "lamb"])
def test_multi_tensor_optimizers(kind):
    from axonml_b200.ops import optim as O
    shapes = [(5,), (33, 7), (70000,), (256, 300)] * 9  # > 24 tensors and > 1 chunk
    ps = [torch.randn(s, device=DEV) for s in shapes]
    gs = [torch.randn(s, device=DEV) for s in shapes]
    ref_p = [p.clone().requires_grad_() for p in ps]
    for p, g in zip(ref_p, gs):
        p.grad = g.clone()
    z = lambda: [torch.zeros_like(p) for p in ps]
    if kind == "sgd":
        opt = torch.optim.SGD(ref_p, lr=0.1, momentum=0.9, weight_decay=0.01, nesterov=True)
        s1 = z()
        for step in range(2):
            opt.step()
            O.multi_tensor("sgd", ps, gs, s1, lr=0.1, momentum=0.9, wd=0.01, nesterov=True,
                           first_step=(step == 0))
    elif kind in ("adam", "adamw"):
        cls = torch.optim.AdamW if kind == "adamw" else torch.optim.Adam
        opt = cls(ref_p, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        s1, s2 = z(), z()
        for step in range(1, 3):
            opt.step()
            O.multi_tensor("adam", ps, gs, s1, s2, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1,
                           bc1=1 - 0.9 ** step, bc2=1 - 0.95 ** step, adamw=(kind == "adamw"))
    elif kind == "rmsprop":
        opt = torch.optim.RMSprop(ref_p, lr=1e-2, alpha=0.99, eps=1e-8, momentum=0.5, centered=True)
        s1, s2, s3 = z(), z(), z()
        for step in range(2):
            opt.step()
            O.multi_tensor("rmsprop", ps, gs, s1, s2, s3, lr=1e-2, alpha=0.99, eps=1e-8,
                           momentum=0.5, centered=True)
    else:
        s1, s2, s3 = z(), z(), z()
        m = [torch.zeros_like(p) for p in ps]
        v = [torch.zeros_like(p) for p in ps]
        for step in range(1, 3):
            norms = torch.zeros(2 * len(ps), device=DEV)
            hp = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-6, wd=0.01, bc1=1 - 0.9 ** step,
                      bc2=1 - 0.999 ** step)
            O.multi_tensor("lamb1", ps, gs, s1, s2, s3, norms=norms, **hp)
            O.multi_tensor("lamb2", ps, gs, s1, s2, s3, norms=norms, **hp)
            with torch.no_grad():
                for i, (p, g) in enumerate(zip(ref_p, gs)):
                    m[i] = 0.9 * m[i] + 0.1 * g
                    v[i] = 0.999 * v[i] + 0.001 * g * g
                    r = (m[i] / hp["bc1"]) / ((v[i] / hp["bc2"]).sqrt() + 1e-6) + 0.01 * p
                    pn, rn = p.norm(), r.norm()
                    trust = pn / rn if pn > 0 and rn > 0 else 1.0
                    p -= 1e-2 * trust * r
    for p, r in zip(ps, ref_p):
        close(p, r.detach(), 1e-5, 1e-4)


def test_grad_sumsq_and_unscale():
    from axonml_b200.ops import optim as O
    gs = [torch.randn(n, device=DEV).bfloat16() for n in (3, 1000, 70001)]
    ss = O.grad_sumsq(gs)
    ref = sum((g.float() ** 2).sum() for g in gs)
    close(ss[0], ref, 1e-2, 1e-3)
    inv = torch.tensor([0.5], device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    fg = [torch.randn(100, device=DEV), torch.randn(5, device=DEV)]
    want = [g * 0.5 for g in fg]
    O.multi_tensor("unscale_check", None, fg, inv_scale=inv, norms=flag)
    assert flag.item() == 0
    for a, b in zip(fg, want):
        close(a, b, 1e-6, 1e-6)
    fg[1][2] = float("inf")
    O.multi_tensor("unscale_check", None, fg, inv_scale=inv, norms=flag)
    assert flag.item() == 1


def test_jit_nvrtc_fused_elementwise_matches_interpreter(kernel_status):
    """A traced elementwise graph compiled with NVRTC for this GPU and launched through the driver
    API gives what the CPU interpreter gives."""
    from axonml_b200 import jit
    from axonml_b200.jit import nvrtc
    if not nvrtc.available():
        pytest.skip("cuda-python bindings not importable")

    def f(tr):
        a, b = tr.input("a", [4096]), tr.input("b", [4096])
        y = a.mul(b).add_scalar(0.5).tanh().mul_scalar(2.0).relu()
        return tr.output("y", y)
    g = jit.trace(f)
    a, b = torch.randn(4096, device="cuda"), torch.randn(4096, device="cuda")
    ref = jit.interpret(g, {"a": a.cpu(), "b": b.cpu()})["y"]
    out = jit.compile_graph(g).run_tensors({"a": a, "b": b})["y"]
    assert out.is_cuda
    assert (out.cpu() - ref).abs().max().item() < 2e-3


def test_kernels_do_not_write_outside_their_outputs(kernel_status):
    """Outputs carved out of canary-padded allocations (a stand-in for a memory checker): ragged
    sizes for the elementwise kernels, non-multiple-of-tile GEMM shapes, padded vocabulary columns
    in the cross-entropy backward, pooling with a window that hangs over the border."""
    from axonml_b200 import _native as N
    from axonml_b200.ops.gemm import gemm_bf16
    from axonml_b200.utils.canary import guarded
    L, st = N.cuda(), N.stream_ptr()
    torch.manual_seed(0)
    for n in (1, 7, 33, 1000, 4097):
        x = torch.randn(n, device="cuda").bfloat16()
        y = guarded((n,), torch.bfloat16)
        assert L.ax_unary(1, 8, N.ptr(x), N.ptr(y.tensor), N.c_int64(n), N.c_float(0.0), N.c_float(0.0), st) == 0      # GELU
        z = guarded((n,), torch.bfloat16)
        assert L.ax_binary(1, 2, N.ptr(x), N.ptr(x), N.ptr(z.tensor), N.c_int64(n), N.c_float(0.0), st) == 0            # mul
        torch.cuda.synchronize()
        y.check(f"unary n={n}"); z.check(f"binary n={n}")
        assert torch.allclose(z.tensor.float(), (x.float() ** 2).bfloat16().float(), atol=1e-2, rtol=1e-2)
    for (m, nn_, k) in ((128, 128, 64), (200, 136, 72), (1, 8, 8), (384, 520, 264)):
        a = torch.randn(m, k, device="cuda").bfloat16()
        b = torch.randn(nn_, k, device="cuda").bfloat16()
        out = guarded((m, nn_), torch.bfloat16)
        gemm_bf16(a, b, out=out.tensor)
        torch.cuda.synchronize()
        out.check(f"gemm {m}x{nn_}x{k}")
        assert torch.allclose(out.tensor.float(), a.float() @ b.float().t(), atol=0.5, rtol=5e-2)
    rows, D = 37, 1024
    x = torch.randn(rows, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    y = guarded((rows, D), torch.bfloat16)
    mean, rstd = guarded((rows,), torch.float32), guarded((rows,), torch.float32)
    assert L.ax_norm_fwd(0, 1, 1, N.ptr(x), N.ptr(None), N.ptr(w), N.ptr(w), N.ptr(y.tensor), N.ptr(None), N.ptr(mean.tensor),
                         N.ptr(rstd.tensor), rows, D, N.c_float(1e-5), st) == 0
    rows, V, stride = 5, 1003, 1024
    logits = torch.randn(rows, stride, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    lse = torch.logsumexp(logits[:, :V].float(), -1)
    dl = guarded((rows, stride), torch.bfloat16)
    assert L.ax_ce_bwd(1, N.ptr(logits), N.ptr(tgt), N.ptr(lse), N.ptr(None), 0, N.c_float(1.0), N.ptr(dl.tensor), rows, V,
                       stride, N.c_int64(stride), N.c_int64(-100), st) == 0
    n_, h, w_, c = 2, 7, 9, 16
    xp = torch.randn(n_, h, w_, c, device="cuda").bfloat16()
    ho, wo = (h + 2 - 3) // 2 + 1, (w_ + 2 - 3) // 2 + 1
    yp, ip = guarded((n_, ho, wo, c), torch.bfloat16), guarded((n_, ho, wo, c), torch.uint8)
    assert L.ax_maxpool2d_fwd(N.ptr(xp), N.ptr(yp.tensor), N.ptr(ip.tensor), n_, h, w_, c, 3, 2, 1, st) == 0
    dxp = guarded((n_, h, w_, c), torch.bfloat16)
    assert L.ax_maxpool2d_bwd(N.ptr(yp.tensor), N.ptr(ip.tensor), N.ptr(dxp.tensor), n_, h, w_, c, 3, 2, 1, st) == 0
    torch.cuda.synchronize()
    for g, what in ((y, "norm y"), (mean, "norm mean"), (rstd, "norm rstd"), (dl, "ce dlogits"), (yp, "pool y"),
                    (ip, "pool idx"), (dxp, "pool dx")):
        g.check(what)
    assert float(dl.tensor[:, V:].abs().max()) == 0.0
    ref = torch.nn.functional.max_pool2d(xp.permute(0, 3, 1, 2).float(), 3, 2, 1).permute(0, 2, 3, 1)
    assert torch.equal(yp.tensor.float(), ref)


@pytest.mark.parametrize("kind,hidden,layers,batch,steps", [("lstm", 128, 1, 1, 128), ("lstm", 48, 2, 3, 17), ("gru", 128, 2, 4, 60),
                                                           ("gru", 20, 1, 2, 9)])
def test_whole_sequence_rnn_kernel_matches_the_step_by_step_path(kind, hidden, layers, batch, steps, kernel_status):
    """LSTM / GRU inference through the one-kernel-per-layer path against the same module evaluated
    step by step in fp32."""
    from axonml_b200 import nn
    torch.manual_seed(0)
    cls = nn.LSTM if kind == "lstm" else nn.GRU
    ref = cls(24, hidden, layers)
    for c in ref.cells:                                  # non-zero biases exercise both bias paths
        c.bias_ih.data.uniform_(-0.2, 0.2)
        c.bias_hh.data.uniform_(-0.2, 0.2)
    import copy
    m = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    for cr, cm in zip(ref.cells, m.cells):               # compare at the weights the GPU module really holds
        for n in ("weight_ih", "weight_hh", "bias_ih", "bias_hh"):
            getattr(cr, n).data.copy_(getattr(cm, n).data.float().cpu())
    x = torch.randn(batch, steps, 24)
    with torch.no_grad():
        want = ref(x)
        got = m(x.to("cuda", torch.bfloat16))
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    assert (got.float().cpu() - want).abs().max().item() < 4e-2
    last = m.last_state[-1]
    h_last = last[0] if kind == "lstm" else last
    assert (h_last.float().cpu() - want[:, -1]).abs().max().item() < 4e-2


def test_lamb_on_a_flat_master_buffer_takes_trust_ratios_per_tensor():
    """A sharded engine hands LAMB one flat fp32 buffer per unit; the multi-tensor kernels run on
    the slices of the tensors inside it (odd starts included), so the result equals LAMB on the
    separate tensors."""
    from axonml_b200 import nn, optim
    from axonml_b200.parallel import FSDP
    torch.manual_seed(0)
    mk = lambda: nn.Sequential(nn.Linear(96, 251), nn.Tanh(), nn.Linear(251, 131), nn.Tanh(), nn.Linear(131, 9))
    m, ref = mk().cuda(), mk().cuda()
    ref.load_state_dict(m.state_dict())
    f = FSDP(m, None, param_dtype=torch.float32)
    opt = optim.LAMB(f.parameters(), 2e-2, weight_decay=0.05)
    ropt = optim.LAMB(list(ref.parameters()), 2e-2, weight_decay=0.05)
    X, Y = torch.randn(3, 16, 96, device="cuda"), torch.randint(0, 9, (3, 16), device="cuda")
    for it in range(3):
        nn.CrossEntropyLoss()(f(X[it]), Y[it]).backward()
        opt.step()
        f.zero_grad()
        nn.CrossEntropyLoss()(ref(X[it]), Y[it]).backward()
        ropt.step()
        ropt.zero_grad()
    sd = f.full_state_dict()
    moved = max((v.detach() - sd0).abs().max().item() for v, sd0 in zip(ref.parameters(), mk().cuda().parameters()))
    err = max((sd[k] - v.detach()).abs().max().item() for k, v in ref.named_parameters())
    assert moved > 1e-3 and err < 1e-5, (moved, err)


def test_a_device_wait_that_runs_out_reports_and_leaves_the_context_usable():
    """The all-reduce kernel of a two-rank communicator is launched for rank 0 only; the buffers of
    both "ranks" are ordinary allocations of this one GPU, so nothing remote is touched and nothing
    else waits.  With the wait budget set to a few milliseconds the start barrier gives up: the
    status word carries the peer-timeout code and the place of the wait, the kernel has run to its
    end, and a complete call (a one-rank communicator) then succeeds."""
    import ctypes
    from axonml_b200 import _native as N
    torch.cuda.synchronize()
    N.check_status()
    slots = N.cuda().ax_comm_signal_slots()
    n = 4096
    bufs = [torch.ones(n, device=DEV), torch.ones(n, device=DEV)]
    sigs = [torch.zeros(max(slots, 64), dtype=torch.int32, device=DEV) for _ in range(2)]
    arr = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    N.set_wait_budget_us(3000)
    try:
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = N.cuda().ax_fused_allreduce(0, arr(bufs), arr(sigs), ctypes.c_void_p(0), 0, 2, ctypes.c_long(0),
                                         ctypes.c_long(n), None, None, ctypes.c_uint(1), None, 4,
                                         N.ptr(N.status_word()), N.stream_ptr())
        assert rc == 0
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 1000.0                  # gave up after milliseconds, not the built-in second
        with pytest.raises(N.KernelTimeout) as ei:
            N.check_status()
        assert ei.value.code == 3 and ei.value.where in (600, 601, 603)
        assert bool((bufs[0] == 1).all())                    # the work was skipped, nothing half-written
    finally:
        N.set_wait_budget_us(0)
    # the same kernel, complete this time
    one = torch.full((n,), 3.0, device=DEV)
    sig1 = torch.zeros(max(slots, 64), dtype=torch.int32, device=DEV)
    rc = N.cuda().ax_fused_allreduce(0, arr([one]), arr([sig1]), ctypes.c_void_p(0), 0, 1, ctypes.c_long(0),
                                     ctypes.c_long(n), None, None, ctypes.c_uint(1), None, 4,
                                     N.ptr(N.status_word()), N.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    N.check_status()
    assert bool((one == 3).all())


def test_an_mbarrier_wait_that_runs_out_is_reported(kernel_status):
    """A GEMM whose wait budget is far below the time its loads need still terminates and reports
    through the status word (or simply succeeds when every wait was served in time); either way
    the next GEMM with the normal budget is correct."""
    from axonml_b200 import _native as N
    from axonml_b200.ops.gemm import gemm_bf16
    a = torch.randn(512, 512, device=DEV).bfloat16()
    b = torch.randn(512, 512, device=DEV).bfloat16()
    torch.cuda.synchronize()
    N.set_wait_budget_us(1)
    try:
        gemm_bf16(a, b)
        torch.cuda.synchronize()
        try:
            N.check_status()
        except N.KernelTimeout as e:
            assert e.code == 1
    finally:
        N.set_wait_budget_us(0)
    c = gemm_bf16(a, b)
    close(c, a.float() @ b.float().t(), atol=0.02 * 512 ** 0.5, rtol=2e-2)


def test_fsdp_cpu_offload_on_the_gpu_matches_device_resident_masters(kernel_status):
    """One rank, bf16 compute: with the master shards and optimizer state in pinned host memory the
    parameters after three steps equal those of the device-resident run."""
    from axonml_b200 import nn, optim
    from axonml_b200.parallel import FSDP
    from axonml_b200.parallel.fsdp import CPUOffload
    outs = []
    for off in (CPUOffload.None_, CPUOffload.Params):
        torch.manual_seed(0)
        m = nn.Sequential(nn.Linear(64, 128), nn.Tanh(), nn.Linear(128, 64)).to("cuda", torch.bfloat16)
        f = FSDP(m).cpu_offload(off)
        opt = optim.AdamW(f.parameters(), 1e-2)
        g = torch.Generator().manual_seed(5)
        X = torch.randn(3, 32, 64, generator=g).cuda().bfloat16()
        for it in range(3):
            f(X[it]).float().pow(2).mean().backward()
            opt.step()
            f.zero_grad()
        if off is not CPUOffload.None_:
            assert all(p.device.type == "cpu" and p.is_pinned() for p in f.parameters())
        outs.append({k: v.float().cpu() for k, v in f.full_state_dict().items()})
    for k in outs[0]:
        assert torch.allclose(outs[0][k], outs[1][k], atol=2e-3, rtol=2e-3), k


@pytest.mark.parametrize("M,N,K", [(1024, 1024, 1024), (129, 257, 65), (7, 5, 3), (300, 1000, 2000), (128, 128, 16)])
def test_sgemm_f32_has_fp32_accuracy(M, N, K):
    """The fp32 GEMM of the backend trait keeps fp32 products: the reference's tolerance for its
    cuBLAS sgemm test (atol 1e-3, rtol 1e-2) against a float64 product, far inside what bf16
    operands could give."""
    from axonml_b200.core.backends import CudaBackend
    a = torch.randn(M, K, device=DEV)
    b = torch.randn(K, N, device=DEV)
    c = CudaBackend(0).gemm_f32(a, b)
    ref = (a.double() @ b.double()).float()
    assert c.dtype == torch.float32
    close(c, ref, atol=1e-3, rtol=1e-2)
    assert (c - ref).abs().max().item() < 2e-4 * K ** 0.5


def test_sgemm_f32_batched():
    from axonml_b200.core.backends import CudaBackend
    a = torch.randn(5, 70, 33, device=DEV)
    b = torch.randn(5, 33, 90, device=DEV)
    c = CudaBackend(0).gemm_batched_f32(a, b)
    close(c, torch.bmm(a.double(), b.double()).float(), atol=1e-3, rtol=1e-2)
    c2 = CudaBackend(0).gemm_batched_f32(list(a), list(b))
    assert torch.equal(c, c2)


def test_adam_bias_correction_does_not_run_ahead_after_skipped_steps(kernel_status):
    """With a GradScaler the decision to skip a step is taken on the device.  A skipped step must
    not count for the bias corrections: after overflow, good, good steps the parameters equal those
    of two plain steps."""
    from axonml_b200 import optim
    torch.manual_seed(0)
    w0 = torch.randn(4096, device=DEV)
    g1, g2 = torch.randn(4096, device=DEV), torch.randn(4096, device=DEV)
    ref = torch.nn.Parameter(w0.clone())
    o_ref = torch.optim.Adam([ref], 1e-2)
    for g in (g1, g2):
        ref.grad = g.clone()
        o_ref.step()
    p = torch.nn.Parameter(w0.clone())
    opt = optim.Adam([p], 1e-2)
    scaler = optim.GradScaler.with_scale(8.0)
    bad = g1.clone()
    bad[7] = float("inf")
    for g in (bad, g1, g2):
        opt.zero_grad()
        p.grad = g * scaler.get_scale()          # what backward of the scaled loss would leave
        scaler.step(opt)
        scaler.update()
    close(p.detach(), ref.detach(), atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels_last", [False, True])
@pytest.mark.parametrize("k,s,p", [(2, 2, 0), (3, 2, 1), (3, 1, 1), ((2, 3), (1, 2), (1, 0))])
def test_avg_pool2d_kernel_forward_backward(dtype, channels_last, k, s, p):
    """AvgPool2d kernels (divisor = pixels inside the image) against torch's
    count_include_pad=False in fp32, values and input gradient, both memory layouts."""
    from axonml_b200.ops.pool import avg_pool2d
    x = torch.randn(3, 10, 13, 11, device=DEV).to(dtype)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    x.requires_grad_()
    y = avg_pool2d(x, k, s, p)
    xr = x.detach().float().cpu().contiguous().requires_grad_()       # reference on the CPU, plain layout
    yr = F.avg_pool2d(xr, k, s, p, count_include_pad=False)
    g = torch.randn_like(yr)
    y.backward(g.to(DEV).to(dtype))
    yr.backward(g)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    close(y.cpu(), yr, tol, tol)
    close(x.grad.cpu(), xr.grad, tol, tol)
    y2 = avg_pool2d(x.detach(), k, s, p, count_include_pad=True)
    close(y2.cpu(), F.avg_pool2d(xr.detach(), k, s, p, count_include_pad=True), tol, tol)


@pytest.mark.parametrize("out", [(1, 1), (7, 7), (3, 5), (4, 2)])
@pytest.mark.parametrize("channels_last", [False, True])
def test_adaptive_avg_pool2d_kernel(out, channels_last):
    """Adaptive pooling kernels against the same window rule written with averaging matrices
    (the CPU path of the op), forward and backward; sizes that do not divide included."""
    from axonml_b200.ops.pool import adaptive_avg_pool2d
    x = torch.randn(2, 6, 14, 15, device=DEV)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    x.requires_grad_()
    y = adaptive_avg_pool2d(x, out)
    xr = x.detach().cpu().requires_grad_()
    yr = adaptive_avg_pool2d(xr, out)
    g = torch.randn_like(yr)
    y.backward(g.to(DEV))
    yr.backward(g)
    close(y.cpu(), yr, 1e-5, 1e-5)
    close(x.grad.cpu(), xr.grad, 1e-5, 1e-5)
    if 14 % out[0] == 0 and 15 % out[1] == 0:
        close(y.cpu(), F.adaptive_avg_pool2d(xr.detach(), out), 1e-5, 1e-5)


def test_avg_pool1d_kernel():
    from axonml_b200 import nn
    x = torch.randn(4, 5, 37, device=DEV, requires_grad=True)
    y = nn.AvgPool1d.with_options(4, 3, 1)(x)
    xr = x.detach().requires_grad_()
    yr = F.avg_pool1d(xr, 4, 3, 1, count_include_pad=False)
    close(y, yr, 1e-5, 1e-5)
    y.sum().backward(); yr.sum().backward()
    close(x.grad, xr.grad, 1e-5, 1e-5)


def _softmax_like_graph():
    from axonml_b200 import jit

    def f(tr):
        x, b, m = tr.input("x", [64, 300]), tr.input("b", [300]), tr.input("m", [64, 1])
        z = x.add(b)                                   # implicit broadcast of a row vector
        e = z.sub(z.max_axis(1, True)).exp()
        p = e.div(e.sum_axis(1, True))                 # two reductions fused with their producers
        w = p.where(m.gt(0.0), p.mul_scalar(0.0))      # Where on a broadcast comparison
        t = w.transpose(0, 1).reshape([300, 64])
        tr.output("p", w)
        tr.output("t", t)
        tr.output("tot", w.sum())
        tr.output("mean0", w.mean_axis(0))
        tr.output("mm", w.matmul(t))
        tr.output("mask", m.gt(0.0).broadcast([64, 300]))
    return jit.trace(f)


def test_jit_lowers_reductions_broadcast_where_and_matmul_to_generated_kernels(kernel_status):
    """A graph far outside the one-kernel case (row-vector broadcast, two per-axis reductions, a full
    sum, Where, Transpose + Reshape, MatMul, a boolean output) runs as generated kernels and gives
    what the interpreter gives on the CPU."""
    from axonml_b200 import jit
    from axonml_b200.jit import nvrtc
    if not nvrtc.available():
        pytest.skip("cuda-python bindings not importable")
    g = _softmax_like_graph()
    x, b, m = torch.randn(64, 300), torch.randn(300), torch.randn(64, 1)
    ref = jit.interpret(g, {"x": x, "b": b, "m": m})
    fn = jit.JitCompiler.new().compile(g)
    out = fn.run_tensors({"x": x.cuda(), "b": b.cuda(), "m": m.cuda()})
    assert fn.uses_generated_kernel() and "__global__" in fn.generated_source()
    for k, r in ref.items():
        o = out[k]
        assert o.is_cuda and o.dtype == r.dtype and tuple(o.shape) == tuple(r.shape), k
        assert (o.float().cpu() - r.float()).abs().max().item() < 2e-3, k


def test_jit_split_reduction_over_a_large_tensor(kernel_status):
    from axonml_b200 import jit
    from axonml_b200.jit import nvrtc
    if not nvrtc.available():
        pytest.skip("cuda-python bindings not importable")

    def f(tr):
        x = tr.input("x", [1 << 20])
        tr.output("s", x.mul(x).sum())
        tr.output("m", x.abs().mean())
    g = jit.trace(f)
    x = torch.randn(1 << 20, device="cuda")
    out = jit.JitCompiler.new().compile(g).run_tensors({"x": x})
    assert abs(out["s"].item() - (x.double() ** 2).sum().item()) < 1e-3 * (1 << 20) ** 0.5 * 4
    assert abs(out["m"].item() - x.abs().double().mean().item()) < 1e-4


def test_bounds_checked_build_reports_a_wrong_index_instead_of_using_it():
    """The debug build of the kernel library (``AXONML_BOUNDS=1``): its self-test walks one element
    past an extent through the checked accessor, which skips the access and records where and which
    index; a token id outside the embedding table and a class index outside the vocabulary are
    reported the same way; correct calls leave the record empty and give the usual results."""
    import os
    import subprocess
    import sys
    prog = r'''
import ctypes, torch
from axonml_b200 import _native as N
assert N.bounds_build() and N.cuda().ax_bounds_enabled() == 1
assert N.bounds_report() is None
buf = torch.zeros(1000 + 64, device="cuda")
assert N.cuda().ax_bounds_selftest(N.ptr(buf), ctypes.c_long(1000), N.stream_ptr()) == 0
r = N.bounds_report()
assert r == {"code": 4, "where": 9000, "index": 1000, "extent": 1000}, r
assert bool((buf[:1000] == 1).all()) and bool((buf[1000:] == 0).all())      # the stray access was skipped
assert N.bounds_report() is None                                            # reading clears the record
# correct calls: no record, right values
from axonml_b200.ops import elementwise as E
from axonml_b200.ops.gemm import gemm_bf16, sgemm_f32
x = torch.randn(4099, device="cuda")
assert torch.allclose(E.unary(x, "relu"), torch.relu(x))
a, b = torch.randn(300, 256, device="cuda").bfloat16(), torch.randn(512, 256, device="cuda").bfloat16()
assert (gemm_bf16(a, b).float() - a.float() @ b.float().t()).abs().max().item() < 0.5
af, bf = torch.randn(70, 33, device="cuda"), torch.randn(33, 90, device="cuda")
assert torch.allclose(sgemm_f32(af, bf), af @ bf, atol=1e-4)
assert N.bounds_report() is None
# a token id outside the table: reported, and the row comes back as zeros
from axonml_b200 import nn
emb = nn.Embedding(10, 8).cuda()
out = emb(torch.tensor([[1, 12, 3]], device="cuda"))
r = N.bounds_report()
assert r is not None and r["where"] == 2000 and r["index"] == 12 and r["extent"] == 10, r
assert bool((out[0, 1] == 0).all())
print("BOUNDS-OK")
'''
    env = dict(os.environ, AXONML_BOUNDS="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", prog], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "BOUNDS-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.parametrize("rows,D", [(3000, 264), (1500, 1000), (4096, 2048), (2000, 4096), (1200, 5120), (700, 8192)])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("with_res", [False, True])
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_norm_forward_single_pass_widths(rows, D, rms, with_res, wdtype):
    """Many bf16 rows take the forward that keeps a row in registers: every width class (ragged
    last vector included), both norms, with and without the fused residual add, bf16 and fp32
    weights, against fp32 torch maths; the saved statistics too."""
    from axonml_b200 import _native as N
    x = torch.randn(rows, D, device=DEV).bfloat16()
    r = torch.randn(rows, D, device=DEV).bfloat16() if with_res else None
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(wdtype)
    b = None if rms else (0.1 * torch.randn(D, device=DEV)).to(wdtype)
    y, h = torch.empty_like(x), (torch.empty_like(x) if with_res else None)
    mean, rstd = torch.empty(rows, device=DEV), torch.empty(rows, device=DEV)
    rc = N.cuda().ax_norm_fwd(int(rms), 1, 1 if wdtype == torch.bfloat16 else 0, N.ptr(x), N.ptr(r), N.ptr(w), N.ptr(b),
                              N.ptr(y), N.ptr(h), N.ptr(mean), N.ptr(rstd), rows, D, N.c_float(1e-5), N.stream_ptr())
    assert rc == 0
    hf = (x.float() + r.float()).bfloat16().float() if with_res else x.float()
    if rms:
        ref = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        close(rstd, torch.rsqrt(hf.pow(2).mean(-1) + 1e-5), 1e-3, 1e-3)
    else:
        ref = F.layer_norm(hf, (D,), w.float(), b.float(), 1e-5)
        close(mean, hf.mean(-1), 1e-3, 1e-3)
        close(rstd, torch.rsqrt(hf.var(-1, unbiased=False) + 1e-5), 1e-3, 1e-3)
    close(y, ref, 3e-2, 2e-2)
    if with_res:
        assert torch.equal(h.float(), hf)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_vocab_parallel_cross_entropy_kernels_on_two_slices(dtype, kernel_status):
    """The vocabulary-parallel loss kernels, with the two ranks' slices evaluated one after the other
    on one GPU: statistics per slice, combined as the collective would, equal the loss over the
    whole vocabulary; the backward of each slice with the global log-sum-exp gives the slices of
    the full gradient.  Ignored rows, a padded last slice and targets on either slice included."""
    from axonml_b200 import _native as N
    T, V0, V1, pad = 300, 1000, 920, 8          # second slice: 920 real classes in 928 columns
    V = V0 + V1
    logits = torch.randn(T, V0 + V1 + pad, device=DEV).to(dtype)
    target = torch.randint(0, V, (T,), device=DEV)
    target[::17] = -100
    ref_in = logits[:, :V].float().requires_grad_()
    ref = F.cross_entropy(ref_in, target, ignore_index=-100)
    ref.backward()
    code = 1 if dtype == torch.bfloat16 else 0
    slices = [(logits[:, :V0].contiguous(), 0, V0, V0), (logits[:, V0:].contiguous(), V0, V1, V1 + pad)]
    stats, locals_ = [], []
    for sl, start, nvalid, width in slices:
        lt = target - start
        lt = torch.where((lt >= 0) & (lt < nvalid), lt, torch.full_like(lt, -1))
        lt = torch.where(target != -100, lt, torch.full_like(lt, -100)).contiguous()
        st = torch.empty(T, 4, device=DEV)
        assert N.cuda().ax_vp_ce_stats(code, N.ptr(sl), N.ptr(lt), N.ptr(st), T, nvalid, N.c_int64(sl.stride(0)), N.stream_ptr()) == 0
        stats.append(st); locals_.append(lt)
    allst = torch.stack(stats)
    m = allst[..., 0].max(0).values
    lse = (m + (allst[..., 1] * (allst[..., 0] - m).exp()).sum(0).log()).contiguous()
    valid = target != -100
    loss = torch.where(valid, lse - allst[..., 2].sum(0), torch.zeros_like(lse)).sum() / valid.sum()
    assert abs(loss.item() - ref.item()) < (1e-4 if dtype == torch.float32 else 2e-2)
    scale = (1.0 / valid.sum().float()).reshape(1).contiguous()
    grads = []
    for (sl, start, nvalid, width), lt in zip(slices, locals_):
        g = torch.full_like(sl, 7.0)
        assert N.cuda().ax_vp_ce_bwd(code, N.ptr(sl), N.ptr(lt), N.ptr(lse), N.ptr(scale), N.c_float(1.0), N.ptr(g), T, nvalid,
                                     width, N.c_int64(sl.stride(0)), N.c_int64(-100), N.stream_ptr()) == 0
        grads.append(g)
    full = torch.cat(grads, 1)
    tol = 1e-6 if dtype == torch.float32 else 2e-4
    close(full[:, :V], ref_in.grad, tol, 2e-2)
    assert bool((full[:, V:] == 0).all())                       # padded columns get a zero gradient


@pytest.mark.gpu
def test_cuda_kernels_facade_and_device_queries():
    from axonml_b200 import core
    from axonml_b200.core import backends as B
    assert B.is_available() and B.device_count() >= 1 and B.is_device_available(0) and not B.is_device_available(64)
    caps = B.get_capabilities(0)
    assert caps.sm_count > 0 and caps.total_memory > 0 and caps.supports_bf16
    k = core.CudaKernels.load(0)
    assert k.has("ax_norm_bwd_noalloc") and not k.has("ax_no_such_entry") and k.launch_config(1000).grid_dim == (4, 1, 1)
    x = torch.linspace(-2, 2, 4096, device="cuda")
    assert torch.allclose(k.launch_elementwise("relu", x), torch.relu(x))
    assert torch.allclose(k.launch_elementwise("add", x, x), 2 * x)
    with pytest.raises(core.CudaError):
        k.launch_elementwise("conv9d", x)
    with pytest.raises(core.CudaError):
        core.CudaKernels.load(64)
    mem = core.GpuMemory.of(x)
    assert mem.backend_type() is core.BackendType.Cuda and mem.size() == 4096 * 4
    s = core.GpuStream.current(0)
    assert s.backend_type() is core.BackendType.Cuda
    s.synchronize()
