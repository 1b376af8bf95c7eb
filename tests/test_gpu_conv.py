"""Implicit-GEMM convolution kernel against the fp32 torch convolution of the same bf16-rounded
operands: forward (bias, ReLU), data gradient, ragged tile edges, 1x1 and 3x3 filters."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

CASES = [
    # N, Cin, H, W, Cout, k, pad
    (8, 64, 56, 56, 64, 3, 1),
    (4, 128, 28, 28, 128, 3, 1),
    (4, 256, 14, 14, 256, 3, 1),
    (32, 512, 7, 7, 512, 3, 1),
    (8, 64, 56, 56, 128, 1, 0),
    (2, 64, 13, 17, 192, 3, 1),
    (3, 128, 9, 9, 64, 5, 2),
    (2, 64, 20, 20, 64, 3, 0),
]


@pytest.mark.parametrize("case", CASES)
def test_conv_fprop_matches_fp32_reference(case, kernel_status):
    from axonml_b200.ops import conv_igemm as CI
    n, cin, h, w, cout, k, pad = case
    torch.manual_seed(0)
    x = torch.randn(n, cin, h, w, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, k, k, device="cuda") * (2.0 / (cin * k * k)) ** 0.5)
    b = torch.randn(cout, device="cuda")
    assert CI.supported(x, wt, (1, 1), (pad, pad))
    y = CI.fprop(x, CI._ohwi(wt), b, (pad, pad), "relu")
    ref = F.relu(F.conv2d(x.float(), wt.bfloat16().float(), b, 1, pad))
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    err = (y.float() - ref).abs().max().item()
    assert err < 0.03 * max(ref.abs().max().item(), 1.0), err


@pytest.mark.parametrize("case", [CASES[0], CASES[3], CASES[5], CASES[6]])
def test_conv_autograd_matches_torch(case, kernel_status):
    from axonml_b200.ops import conv_igemm as CI
    n, cin, h, w, cout, k, pad = case
    torch.manual_seed(1)
    x = torch.randn(n, cin, h, w, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, k, k, device="cuda") * (2.0 / (cin * k * k)) ** 0.5)
    b = torch.zeros(cout, device="cuda")
    x1, w1, b1 = x.clone().requires_grad_(True), wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
    y = CI.conv2d(x1, w1, b1, (1, 1), (pad, pad))
    g = torch.randn_like(y)
    y.backward(g)
    x2, w2, b2 = x.float().requires_grad_(True), wt.bfloat16().float().requires_grad_(True), b.clone().requires_grad_(True)
    F.conv2d(x2, w2, b2, 1, pad).backward(g.float())
    for a, r, tol in ((x1.grad, x2.grad, 0.03), (w1.grad, w2.grad, 0.05), (b1.grad, b2.grad, 0.02)):
        err = (a.float() - r).abs().max().item()
        assert err < tol * max(r.abs().max().item(), 1.0), err


STRIDED = [
    # N, Cin, H, W, Cout, k, pad, stride
    (8, 64, 56, 56, 128, 3, 1, (2, 2)),
    (4, 128, 28, 28, 256, 1, 0, (2, 2)),
    (3, 64, 13, 17, 128, 3, 1, (2, 2)),
    (2, 64, 16, 15, 64, 5, 2, (2, 2)),
    (4, 64, 12, 12, 64, 2, 0, (2, 2)),
    (2, 64, 15, 22, 64, 3, 1, (2, 1)),
    (2, 128, 14, 14, 64, 3, 0, (1, 2)),
]


@pytest.mark.parametrize("case", STRIDED)
def test_strided_conv_forward_and_gradients_match_fp32_reference(case, kernel_status):
    """Strided convolutions read the input through parity views; their data gradient runs one
    launch per parity class of the input pixels, their weight gradient the pixel-reduction kernel
    over the same views."""
    from axonml_b200 import _native
    from axonml_b200.ops import conv_igemm as CI
    n, cin, h, w, cout, k, pad, stride = case
    torch.manual_seed(2)
    x = torch.randn(n, cin, h, w, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, k, k, device="cuda") * (2.0 / (cin * k * k)) ** 0.5)
    b = torch.randn(cout, device="cuda")
    assert CI.supported(x, wt, stride, (pad, pad))
    x1, w1, b1 = x.clone().requires_grad_(True), wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
    before = _native.launch_count()
    y = CI.conv2d(x1, w1, b1, stride, (pad, pad))
    x2, w2, b2 = x.float().requires_grad_(True), wt.bfloat16().float().requires_grad_(True), b.clone().requires_grad_(True)
    ref = F.conv2d(x2, w2, b2, stride, pad)
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    assert (y.float() - ref).abs().max().item() < 0.03 * max(ref.abs().max().item(), 1.0)
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float())
    assert _native.launch_count() >= before + 3
    for a, r, tol in ((x1.grad, x2.grad, 0.03), (w1.grad, w2.grad, 0.05), (b1.grad, b2.grad, 0.02)):
        err = (a.float() - r).abs().max().item()
        assert err < tol * max(r.abs().max().item(), 1.0), err


def test_resnet_block_uses_the_kernel(kernel_status):
    """Conv2d layers of a channels-last bf16 ResNet stage go through the implicit-GEMM path."""
    from axonml_b200 import _native, nn
    conv = nn.Conv2d(64, 64, 3, 1, 1, bias=False).cuda()
    x = torch.randn(4, 64, 56, 56, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    before = _native.launch_count()
    y = conv(x)
    assert _native.launch_count() > before
    ref = F.conv2d(x.float(), conv.weight.bfloat16().float(), None, 1, 1)
    assert (y.float() - ref).abs().max().item() < 0.03 * ref.abs().max().item()


@pytest.mark.parametrize("shape,relu,res", [((8, 64, 56, 56), True, False), ((4, 128, 28, 28), True, True),
                                              ((16, 512, 7, 7), False, False), ((2, 192, 9, 11), True, True)])
def test_batchnorm_train_fwd_bwd_matches_fp32_reference(shape, relu, res, kernel_status):
    from axonml_b200.ops import batchnorm as BN
    torch.manual_seed(0)
    n, c, h, w = shape
    x = (torch.randn(shape, device="cuda") * 2 + 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    r = torch.randn(shape, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last) if res else None
    g = torch.randn(shape, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    wt, b = torch.rand(c, device="cuda") + 0.5, torch.randn(c, device="cuda")
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    x1, w1, b1 = x.clone().requires_grad_(True), wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
    r1 = r.clone().requires_grad_(True) if res else None
    y = BN.batch_norm(x1, w1, b1, rm, rv, True, 0.1, 1e-5, relu, r1)
    y.backward(g)
    # fp32 reference
    x2, w2, b2 = x.float().requires_grad_(True), wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
    r2 = r.float().requires_grad_(True) if res else None
    rm2, rv2 = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    z = torch.nn.functional.batch_norm(x2, None, None, w2, b2, True, 0.0, 1e-5)
    if res:
        z = z + r2
    if relu:
        z = torch.relu(z)
    z.backward(g.float())
    xf = x.float()
    rm2.mul_(0.9).add_(xf.mean((0, 2, 3)), alpha=0.1)
    rv2.mul_(0.9).add_(xf.var((0, 2, 3), unbiased=False), alpha=0.1)
    assert (y.float() - z).abs().max().item() < 0.05
    assert (rm - rm2).abs().max().item() < 1e-3 and (rv - rv2).abs().max().item() < 1e-2
    assert (x1.grad.float() - x2.grad).abs().max().item() < 0.05 * max(x2.grad.abs().max().item(), 1e-3) + 2e-3
    assert (w1.grad - w2.grad).abs().max().item() < 0.02 * w2.grad.abs().max().item() + 0.05
    assert (b1.grad - b2.grad).abs().max().item() < 0.02 * b2.grad.abs().max().item() + 0.05
    if res:
        assert (r1.grad.float() - r2.grad).abs().max().item() < 0.02


def test_batchnorm_eval_and_maxpool(kernel_status):
    from axonml_b200.ops import batchnorm as BN
    torch.manual_seed(1)
    x = torch.randn(4, 64, 20, 20, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    wt, b = torch.rand(64, device="cuda") + 0.5, torch.randn(64, device="cuda")
    rm, rv = torch.randn(64, device="cuda") * 0.1, torch.rand(64, device="cuda") + 0.5
    y = BN.batch_norm(x, wt, b, rm, rv, False, 0.1, 1e-5, True, None)
    ref = torch.relu(torch.nn.functional.batch_norm(x.float(), rm, rv, wt, b, False, 0.0, 1e-5))
    assert (y.float() - ref).abs().max().item() < 0.05
    for (k, s, p) in ((3, 2, 1), (2, 2, 0)):
        x1 = x.clone().requires_grad_(True)
        o = BN.max_pool2d(x1, k, s, p)
        g = torch.randn_like(o)
        o.backward(g)
        x2 = x.float().requires_grad_(True)
        o2 = torch.nn.functional.max_pool2d(x2, k, s, p)
        o2.backward(g.float())
        assert torch.equal(o.float(), o2)
        assert (x1.grad.float() - x2.grad).abs().max().item() < 0.02


@pytest.mark.parametrize("cin,cout,k,stride,pad,hw", [(3, 64, 7, 2, 3, 64), (3, 32, 3, 1, 1, 33), (1, 16, 5, 2, 2, 28), (4, 64, 7, 2, 3, 224)])
def test_thin_input_convolution_im2col_gemm(cin, cout, k, stride, pad, hw, kernel_status):
    """The RGB-stem path (im2col kernel + tcgen05 GEMM) against the fp32 convolution, with the
    gradients of weight and bias."""
    from axonml_b200.ops import conv_igemm as CI
    torch.manual_seed(0)
    n = 4
    x = torch.randn(n, cin, hw, hw, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(cout, cin, k, k, device="cuda") * 0.1).requires_grad_()
    b = torch.randn(cout, device="cuda").requires_grad_()
    assert CI.thin_supported(x, w, (stride, stride), (pad, pad))
    y = CI.conv2d(x, w, b, (stride, stride), (pad, pad))
    assert y.is_contiguous(memory_format=torch.channels_last)
    wr, br = w.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    ref = F.conv2d(x.float(), wr.bfloat16().float(), br, stride, pad)
    assert y.shape == ref.shape
    assert (y.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item() + 0.05
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float())
    assert (w.grad - wr.grad).abs().max().item() < 0.03 * wr.grad.abs().max().item() + 1e-2
    assert (b.grad - br.grad).abs().max().item() < 0.02 * br.grad.abs().max().item() + 1e-2


@pytest.mark.parametrize("n,cin,l,cout,k,stride,pad", [(4, 64, 200, 128, 3, 1, 1), (2, 128, 333, 64, 5, 2, 2), (8, 64, 64, 64, 1, 1, 0)])
def test_conv1d_runs_on_the_implicit_gemm_kernels(n, cin, l, cout, k, stride, pad, kernel_status):
    """Conv1d as a convolution over an image of height one: forward and all three gradients against
    the fp32 reference, and a second layer on the (channels-last) result without a transpose."""
    from axonml_b200 import _native, nn
    torch.manual_seed(5)
    conv = nn.Conv1d(cin, cout, k, stride, pad).cuda()
    x = torch.randn(n, cin, l, device="cuda").bfloat16().requires_grad_(True)
    before = _native.launch_count()
    y = conv(x)
    assert _native.launch_count() > before and y.shape == (n, cout, (l + 2 * pad - k) // stride + 1)
    g = torch.randn_like(y)
    y.backward(g)
    x2 = x.detach().float().requires_grad_(True)
    w2 = conv.weight.detach().bfloat16().float().requires_grad_(True)
    b2 = conv.bias.detach().clone().requires_grad_(True)
    ref = F.conv1d(x2, w2, b2, stride, pad)
    ref.backward(g.float())
    assert (y.float() - ref).abs().max().item() < 0.03 * max(ref.abs().max().item(), 1.0)
    for a, r, tol in ((x.grad, x2.grad, 0.03), (conv.weight.grad, w2.grad, 0.05), (conv.bias.grad, b2.grad, 0.02)):
        assert (a.float() - r).abs().max().item() < tol * max(r.abs().max().item(), 1.0)
    if cout % 64 == 0:
        z = nn.Conv1d(cout, 64, 3, 1, 1).cuda()(y.detach())          # consumes the strided view directly
        assert z.shape[:2] == (n, 64)
