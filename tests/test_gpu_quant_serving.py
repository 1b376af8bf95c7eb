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


@pytest.mark.parametrize("B,N,K", [(1, 4096, 4096), (3, 500, 14336), (5, 136, 768), (8, 1000, 1024)])
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
