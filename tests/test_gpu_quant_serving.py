"""Quantisation and serving kernels on the GPU: block quantise / dequantise against the C++ CPU
codecs, the dequantising matmul against a dequantise-then-fp32-matmul reference, paged KV write
and decode attention against a dense fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qt", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q4_K"])
def test_dequantize_matches_cpu_codec(qt):
    from axonml_b200.quant import QuantType, dequantize_tensor, quantize_tensor
    t = QuantType[qt]
    x = torch.randn(64, 1024) * 0.02
    q = quantize_tensor(x, t)
    ref = dequantize_tensor(q)
    got = dequantize_tensor(q.to("cuda"))
    assert torch.allclose(got.cpu(), ref, atol=1e-6)
    assert torch.allclose(dequantize_tensor(q.to("cuda"), torch.bfloat16).float().cpu(), ref, atol=2e-3, rtol=1e-2)


@pytest.mark.parametrize("qt,limit", [("Q8_0", 0.01), ("Q4_K", 0.12)])
def test_gpu_quantize_error_and_cpu_readable(qt, limit):
    from axonml_b200.quant import QuantType, dequantize_tensor, quantize_tensor
    t = QuantType[qt]
    x = (torch.randn(128, 2048, device="cuda") * 0.02)
    q = quantize_tensor(x, t)
    assert q.data.is_cuda and q.data.numel() == x.numel() // t.block_size() * t.bytes_per_block()
    y_cpu = dequantize_tensor(q.to("cpu"))                     # the CPU codec reads what the GPU wrote
    rmse = ((y_cpu - x.cpu()) ** 2).mean().sqrt().item() / 0.02
    assert rmse < limit, rmse
    q16 = quantize_tensor(x.bfloat16(), t)
    assert ((dequantize_tensor(q16).cpu() - x.cpu()) ** 2).mean().sqrt().item() / 0.02 < limit * 1.3


@pytest.mark.parametrize("qt", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1"])
def test_gpu_quantize_writes_the_bytes_of_the_cpu_codec(qt):
    """The 32-element formats follow one rule on both devices (scale from the block's extremes,
    round to nearest even), so the GPU's blocks must be the CPU codec's blocks byte for byte; a
    zero block and a constant block exercise the zero-scale branches."""
    from axonml_b200.quant import QuantType, quantize_tensor
    t = QuantType[qt]
    torch.manual_seed(3)
    x = torch.randn(96, 1024) * 0.05
    x[0, :32] = 0.0
    x[1, :32] = 0.7
    ref = quantize_tensor(x, t).data
    got = quantize_tensor(x.cuda(), t).data
    assert got.is_cuda and got.dtype == torch.uint8 and got.numel() == ref.numel()
    differing = (got.cpu() != ref).sum().item()
    assert differing == 0, f"{differing} of {ref.numel()} bytes differ"


@pytest.mark.parametrize("qt", ["Q4_K", "Q8_0"])
@pytest.mark.parametrize("B,N,K", [(1, 128, 256), (8, 768, 4096), (33, 200, 1024), (64, 4096, 1792 // 256 * 256), (100, 384, 512)])
def test_qgemm(qt, B, N, K, kernel_status):
    from axonml_b200.ops.quant import qgemm
    from axonml_b200.quant import QuantType, dequantize_tensor, quantize_tensor
    w = torch.randn(N, K) * 0.05
    q = quantize_tensor(w, QuantType[qt]).to("cuda")
    x = torch.randn(B, K, device="cuda").bfloat16()
    from axonml_b200.ops.quant import tile_weight, untile_weight
    y = qgemm(x, q)
    ref = x.float() @ dequantize_tensor(q).float().t()
    err = (y - ref).abs().max().item()
    assert err < 0.02 * (K ** 0.5) * 0.05 * 4 + 1e-2, err
    qt_ = tile_weight(q)
    assert torch.equal(untile_weight(qt_).data, q.data)
    assert (qgemm(x, qt_) - y).abs().max().item() < 1e-3


@pytest.mark.parametrize("B,N,K", [(1, 4096, 4096), (3, 500, 14336), (5, 136, 768), (8, 1000, 1024),
                                   (1, 4096, 512), (2, 4099, 1792), (1, 768, 4096), (4, 4096, 1024), (1, 4096, 14336),
                                   (2, 30, 256)])
def test_q4k_matrix_vector_kernel(B, N, K, kernel_status, monkeypatch):
    """Decode-sized batches take the dp4a matrix-vector kernel (both weight layouts); the result is
    compared with the fp32 product of the dequantised weights and with the tensor-core kernel."""
    from axonml_b200.ops.quant import qgemm, tile_weight
    from axonml_b200.quant import QuantType, dequantize_tensor, quantize_tensor
    torch.manual_seed(1)
    w = torch.randn(N, K) * 0.05
    q = quantize_tensor(w, QuantType.Q4_K).to("cuda")
    x = torch.randn(B, K, device="cuda").bfloat16()
    ref = x.float() @ dequantize_tensor(q).float().t()
    y = qgemm(x, q)
    tol = 0.01 * (K ** 0.5) * 0.05 * 4 + 1e-2          # int8 activations: about 0.4 % per element
    if B > 4:                                           # larger batches stay on the tensor-core kernel
        tol = 2 * tol + 0.05
    assert y.shape == (B, N) and (y - ref).abs().max().item() < tol
    yt = qgemm(x, tile_weight(q))
    assert (yt - y).abs().max().item() < 1e-4
    yb = qgemm(x, q, out_dtype=torch.bfloat16)            # the matrix-vector kernel writes bf16 itself
    assert yb.dtype == torch.bfloat16 and (yb.float() - y).abs().max().item() <= y.abs().max().item() / 128
    monkeypatch.setenv("AXONML_QGEMV", "0")
    y_tc = qgemm(x, q)
    assert (y_tc - ref).abs().max().item() < 2 * tol + 0.05


@pytest.mark.parametrize("B,N,K", [(1, 18981, 4096), (2, 20000, 1024), (3, 19072, 256), (4, 19000, 1536)])
def test_q80_matrix_vector_kernel(B, N, K, kernel_status, monkeypatch):
    """Wide Q8_0 matrices (an LM head) at decode batch sizes: the shared-memory streaming kernel
    against the fp32 product of the dequantised weights and against the tensor-core kernel."""
    from axonml_b200.ops.quant import qgemm, tile_weight
    from axonml_b200.quant import QuantType, dequantize_tensor, quantize_tensor
    torch.manual_seed(2)
    w = torch.randn(N, K, device="cuda") * 0.05
    q = quantize_tensor(w, QuantType.Q8_0)
    x = torch.randn(B, K, device="cuda").bfloat16()
    ref = x.float() @ dequantize_tensor(q).float().t()
    tol = 0.01 * (K ** 0.5) * 0.05 * 4 + 1e-2
    y = qgemm(x, tile_weight(q))
    assert y.shape == (B, N) and (y - ref).abs().max().item() < tol
    yb = qgemm(x, tile_weight(q), out_dtype=torch.bfloat16)
    assert yb.dtype == torch.bfloat16 and (yb.float() - y).abs().max().item() <= y.abs().max().item() / 128
    monkeypatch.setenv("AXONML_QGEMV", "0")
    y_tc = qgemm(x, tile_weight(q))
    assert (y_tc - ref).abs().max().item() < 2 * tol + 0.05
    assert (y_tc - y).abs().max().item() < 2 * tol + 0.05


def test_paged_kv_and_decode_attention():
    from axonml_b200.ops import paged
    B, Hq, Hkv, D, page, max_pages = 3, 4, 1, 128, 16, 8
    ctx = torch.tensor([37, 5, 100], dtype=torch.int32, device="cuda")
    kc = torch.zeros(64, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    table = torch.randperm(64, device="cuda")[: B * max_pages].view(B, max_pages).int()
    ks, vs, seq, pos = [], [], [], []
    dense = []
    for b in range(B):
        n = int(ctx[b])
        k = torch.randn(n, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(n, Hkv, D, device="cuda").bfloat16()
        dense.append((k, v))
        ks.append(k); vs.append(v)
        seq += [b] * n
        pos += list(range(n))
    paged.kv_write(torch.cat(ks), torch.cat(vs), kc, vc, table, torch.tensor(seq, dtype=torch.int32, device="cuda"),
                   torch.tensor(pos, dtype=torch.int32, device="cuda"), page)
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    out = paged.decode_attention(q, kc, vc, table, ctx, page)
    for b in range(B):
        k, v = dense[b]
        s = torch.einsum("hd,nd->hn", q[b].float(), k[:, 0].float()) / D ** 0.5
        ref = torch.softmax(s, -1) @ v[:, 0].float()
        assert (out[b].float() - ref).abs().max().item() < 3e-2
    # CPU path gives the same numbers
    out_cpu = paged.decode_attention(q.cpu().float(), kc.cpu().float(), vc.cpu().float(), table.cpu(), ctx.cpu(), page)
    assert (out_cpu - out.float().cpu()).abs().max().item() < 3e-2


def _q8_reference(y: torch.Tensor):
    """int8 blocks of 32 of fp32 rows, by the kernels' rule (scale = absmax / 127, nearest even)."""
    B, K = y.shape
    blk = y.view(B, K // 32, 32)
    d = blk.abs().amax(-1, keepdim=True) / 127.0
    q = torch.where(d > 0, torch.round(blk / d.clamp_min(1e-30)), torch.zeros_like(blk))
    return q.view(B, K), d.view(B, K // 32), (d * q.sum(-1, keepdim=True)).view(B, K // 32)


@pytest.mark.parametrize("B,K,wdt", [(1, 4096, torch.float32), (3, 2048, torch.bfloat16), (4, 8192, torch.float32), (2, 160, torch.bfloat16)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_decode_norm_writes_int8_blocks(B, K, wdt, with_residual, kernel_status):
    from axonml_b200.ops import decode as Dc
    torch.manual_seed(0)
    x = torch.randn(B, K, device="cuda").bfloat16()
    r = torch.randn(B, K, device="cuda").bfloat16() if with_residual else None
    w = (torch.rand(K, device="cuda") + 0.5).to(wdt)
    a, stream, h = Dc.rms_norm_q8(x, w, 1e-5, residual=r, want_bf16=True)
    xs = (x.float() + r.float()).bfloat16() if with_residual else x
    assert torch.equal(stream, xs)
    ref = (xs.float() * torch.rsqrt(xs.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float())
    assert (h.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item()
    q, d, s = _q8_reference(h.float())
    assert (a.dx.view(B, -1) - d).abs().max().item() < 1e-6 * d.max().item() + 1e-9
    assert (a.x8.view(B, K).float() - q).abs().max().item() <= 1.0          # a tie may round the other way
    assert (a.x8.view(B, K).float() != q).float().mean().item() < 1e-2       # ties (x * (1/d) against x / d)
    assert (a.sx.view(B, -1) - a.dx.view(B, -1) * a.x8.view(B, K // 32, 32).float().sum(-1)).abs().max().item() < 1e-5
    assert (a.dequantize() - h.float()).abs().max().item() <= d.max().item() * 0.51


def test_decode_swiglu_and_plain_quantiser_write_int8_blocks(kernel_status):
    from axonml_b200.ops import decode as Dc
    torch.manual_seed(1)
    B, F = 3, 1792
    gu = torch.randn(B, 2 * F, device="cuda").bfloat16()
    a = Dc.swiglu_q8(gu)
    y = (torch.nn.functional.silu(gu[:, :F].float()) * gu[:, F:].float()).bfloat16().float()
    assert (a.dequantize() - y).abs().max().item() < 0.02 * y.abs().max().item()
    x = torch.randn(4, 512, device="cuda").bfloat16()
    b = Dc.quantize_rows(x)
    q, d, s = _q8_reference(x.float())
    assert (b.dx.view(4, -1) - d).abs().max().item() < 1e-6 and (b.x8.view(4, 512).float() - q).abs().max().item() <= 1.0
    assert (b.sx.view(4, -1) - s).abs().max().item() < 0.02 * s.abs().max().item() + 1e-4


@pytest.mark.parametrize("B,N,K", [(1, 4096, 4096), (2, 6144, 1024), (4, 500, 14336)])
def test_matrix_vector_kernel_on_int8_from_a_producer(B, N, K, kernel_status):
    """norm -> int8 -> matrix-vector kernel equals norm -> bf16 -> (quantiser + matrix-vector kernel)."""
    from axonml_b200.ops import decode as Dc
    from axonml_b200.ops import norm as Nm
    from axonml_b200.ops.quant import qgemm
    from axonml_b200.quant import QuantType, quantize_tensor
    torch.manual_seed(2)
    wq = quantize_tensor(torch.randn(N, K, device="cuda") * 0.05, QuantType.Q4_K)
    x = torch.randn(B, K, device="cuda").bfloat16()
    w = torch.rand(K, device="cuda") + 0.5
    a, _, h = Dc.rms_norm_q8(x, w, 1e-5, want_bf16=True)
    y = Dc.qgemv(a, wq, out_dtype=torch.float32)
    ref = qgemm(h, wq)                                     # same int8 rule on the same bf16 rows
    assert (y - ref).abs().max().item() < 2e-3 * ref.abs().max().item() + 1e-3
    h2 = Nm.rms_norm(x, w, 1e-5)
    assert (h.float() - h2.float()).abs().max().item() <= 0.02 * h2.float().abs().max().item()


def test_rope_and_kv_write_in_one_launch(kernel_status):
    from axonml_b200.ops import decode as Dc
    from axonml_b200.ops import misc as Mi
    from axonml_b200.ops import paged
    torch.manual_seed(3)
    B, Hq, Hkv, D, page, max_pages = 3, 8, 2, 128, 16, 6
    cos, sin = Mi.rope_tables(256, D, 10000.0, device="cuda")
    qkv = torch.randn(B, Hq + 2 * Hkv, D, device="cuda").bfloat16()
    pos = torch.tensor([5, 33, 80], dtype=torch.int32, device="cuda")
    table = torch.randperm(40, device="cuda")[: B * max_pages].view(B, max_pages).int()
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    kc = torch.zeros(40, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = Dc.rope_kv_write(qkv, cos, sin, pos, kc, vc, table, seq, Hq, Hkv, page)
    ref = Mi.rope_positions(qkv, cos, sin, pos, rot_heads=Hq + Hkv)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    paged.kv_write(ref[:, Hq:Hq + Hkv], ref[:, Hq + Hkv:], kc2, vc2, table, seq, pos, page)
    assert torch.equal(q, ref[:, :Hq].contiguous())
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)


def test_decode_attention_merge_writes_int8_blocks(kernel_status):
    from axonml_b200.ops import decode as Dc
    from axonml_b200.ops import paged
    torch.manual_seed(4)
    B, Hq, Hkv, D, page, max_pages = 2, 8, 2, 128, 16, 8
    kc = torch.randn(32, page, Hkv, D, device="cuda").bfloat16()
    vc = torch.randn(32, page, Hkv, D, device="cuda").bfloat16()
    table = torch.randperm(32, device="cuda")[: B * max_pages].view(B, max_pages).int()
    ctx = torch.tensor([100, 17], dtype=torch.int32, device="cuda")
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    ref = paged.decode_attention(q, kc, vc, table, ctx, page)
    out, a = Dc.decode_attention_q8(q, kc, vc, table, ctx, page)
    assert (out.float() - ref.float()).abs().max().item() < 2e-2
    qq, d, _ = _q8_reference(out.float().view(B, Hq * D))
    assert (a.dx.view(B, -1) - d).abs().max().item() < 1e-6 and (a.x8.view(B, -1).float() - qq).abs().max().item() <= 1.0


def test_fused_decode_step_matches_the_unfused_step(kernel_status, monkeypatch):
    """QuantizedLlama.decode at batch 2 on the fused path against the same step with the fusions off."""
    from axonml_b200.llm import LLaMAConfig
    from axonml_b200.quant import QuantType
    from axonml_b200.server import LLMEngine, QuantizedLlama
    cfg = LLaMAConfig(vocab_size=20000, hidden_size=1024, intermediate_size=2048, num_hidden_layers=2,
                      num_attention_heads=8, num_key_value_heads=4, max_position_embeddings=256)
    model = QuantizedLlama.from_random(cfg, None, device="cuda", std=0.05, proj_type=QuantType.Q4_K)
    prompts = [[(11 * i + j) % 19000 for j in range(20)] for i in range(2)]
    monkeypatch.setenv("AXONML_DECODE_GRAPHS", "0")
    monkeypatch.setenv("AXONML_DECODE_FUSED", "1")
    a = LLMEngine(model, max_batch=2, max_context=64, page_size=16).generate(prompts, 8)
    monkeypatch.setenv("AXONML_DECODE_FUSED", "0")
    b = LLMEngine(model, max_batch=2, max_context=64, page_size=16).generate(prompts, 8)
    # greedy tokens of two numerically close paths: the first tokens agree, later ones may fork at a near-tie
    assert [x[:3] for x in a] == [x[:3] for x in b], (a, b)
