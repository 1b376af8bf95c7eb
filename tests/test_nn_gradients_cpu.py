"""Per-layer gradient checks: every ``nn`` module's backward against central finite differences in
float64 (``torch.autograd.gradcheck``), inputs and parameters alike.  This is the reference's
numerical-gradient methodology (crates/axonml-autograd/src/backward.rs:117-180 and the per-layer
tests of crates/axonml-nn) applied layer by layer."""
import pytest
import torch

from axonml_b200 import nn


def _double(m):
    m = m.double()
    for p in m.parameters():
        p.requires_grad_(True)
    return m


def _check(module, *inputs, fn=None, eps=1e-6, atol=1e-5, rtol=1e-4):
    """gradcheck of ``module(*inputs)`` with respect to the inputs that need a gradient and every
    parameter of the module."""
    module = _double(module)
    params = list(module.parameters())
    diff_in = [x for x in inputs if torch.is_tensor(x) and x.requires_grad]

    def f(*flat):
        n = len(diff_in)
        it = iter(flat[:n])
        args = [next(it) if (torch.is_tensor(x) and x.requires_grad) else x for x in inputs]
        saved = [p.data for p in params]
        for p, v in zip(params, flat[n:]):
            p.data = v.data
        try:
            # run on the tensors handed in, so that finite differences see the parameters move
            out = torch.func.functional_call(module, {k: v for (k, _), v in zip(module.named_parameters(), flat[n:])}, tuple(args))
        finally:
            for p, v in zip(params, saved):
                p.data = v
        out = out[0] if isinstance(out, tuple) else out
        return fn(out) if fn is not None else out

    flat = tuple(diff_in) + tuple(p.detach().clone().requires_grad_() for p in params)
    assert torch.autograd.gradcheck(f, flat, eps=eps, atol=atol, rtol=rtol, nondet_tol=0.0)


def _x(*shape, grad=True):
    return torch.randn(*shape, dtype=torch.float64).requires_grad_(grad)


def test_linear_and_fused_activations():
    for act in (None, "relu", "gelu", "silu", "tanh", "sigmoid"):
        torch.manual_seed(0)
        _check(nn.Linear(5, 4, activation=act), _x(3, 5) + 0.05)


def test_conv_layers():
    torch.manual_seed(1)
    _check(nn.Conv2d(2, 3, 3, stride=1, padding=1), _x(2, 2, 5, 5))
    _check(nn.Conv2d(2, 4, 3, stride=2, padding=1), _x(1, 2, 6, 6))
    _check(nn.Conv1d(2, 3, 3, stride=1, padding=1), _x(2, 2, 7))


def test_normalisation_layers():
    torch.manual_seed(2)
    _check(nn.LayerNorm(6), _x(4, 6))
    _check(nn.RMSNorm(6), _x(4, 6))
    _check(nn.GroupNorm(2, 4), _x(2, 4, 3, 3))
    _check(nn.InstanceNorm2d(3), _x(2, 3, 4, 4))
    bn = nn.BatchNorm1d(5)
    bn.train()
    _check(bn, _x(6, 5))
    bn2 = nn.BatchNorm2d(3)
    bn2.train()
    _check(bn2, _x(4, 3, 3, 3))
    bn2.eval()
    _check(bn2, _x(2, 3, 3, 3))


def test_pooling_layers():
    torch.manual_seed(3)
    _check(nn.AvgPool2d.with_options(3, 2, 1), _x(2, 2, 7, 7))
    _check(nn.AvgPool1d.with_options(3, 2, 1), _x(2, 2, 9))
    _check(nn.AdaptiveAvgPool2d((2, 3)), _x(2, 2, 7, 8))
    # max pooling is piecewise linear: keep the entries of every window apart so that a finite
    # difference step cannot change the arg-max
    base = torch.arange(2 * 2 * 6 * 6, dtype=torch.float64).reshape(2, 2, 6, 6)
    perm = torch.randperm(base.numel()).reshape(base.shape).double()
    _check(nn.MaxPool2d(2), (perm * 0.1).requires_grad_(True))
    _check(nn.MaxPool1d(2), (torch.randperm(24).double().reshape(2, 2, 6) * 0.1).requires_grad_(True))


def test_activation_modules():
    torch.manual_seed(4)
    x = lambda: (_x(3, 7).detach() * 2 + 0.123).requires_grad_(True)      # away from the kinks at 0
    for m in (nn.ReLU(), nn.LeakyReLU(), nn.Sigmoid(), nn.Tanh(), nn.GELU(), nn.SiLU(), nn.ELU(), nn.Identity(),
              nn.Softmax(-1), nn.LogSoftmax(-1)):
        _check(m, x())


def test_embedding_and_attention():
    torch.manual_seed(5)
    ids = torch.tensor([[0, 2, 1], [3, 3, 0]])
    _check(nn.Embedding(4, 5), ids)
    mha = nn.MultiHeadAttention(8, 2)
    mha.eval()
    _check(mha, _x(2, 3, 8), atol=1e-4)


def test_recurrent_layers():
    torch.manual_seed(6)
    for cls in (nn.RNNCell, nn.GRUCell):
        _check(cls(3, 4), _x(2, 3), _x(2, 4))
    _check(nn.LSTMCell(3, 4), _x(2, 3), (_x(2, 4), _x(2, 4)), fn=lambda o: o)
    for cls in (nn.RNN, nn.GRU, nn.LSTM):
        _check(cls(3, 4), _x(2, 5, 3), fn=lambda o: o)


def test_losses():
    torch.manual_seed(7)
    t = torch.randn(4, 3, dtype=torch.float64)
    for m in (nn.MSELoss(), nn.L1Loss(), nn.SmoothL1Loss()):
        _check(m, _x(4, 3), t)
    y = torch.tensor([0, 2, 1, 1])
    _check(nn.CrossEntropyLoss(), _x(4, 3), y)
    _check(nn.NLLLoss(), torch.log_softmax(_x(4, 3).detach(), -1).requires_grad_(True), y)
    p = torch.rand(4, 3, dtype=torch.float64).clamp(0.1, 0.9).requires_grad_(True)
    tt = torch.rand(4, 3, dtype=torch.float64)
    _check(nn.BCELoss(), p, tt)
    _check(nn.BCEWithLogitsLoss(), _x(4, 3), tt)


def test_dropout_in_eval_is_the_identity_and_in_training_scales_its_gradient():
    torch.manual_seed(8)
    d = nn.Dropout(0.5)
    d.eval()
    _check(d, _x(3, 4))
    d.train()
    x = _x(50, 40)
    y = d(x)
    y.sum().backward()
    kept = y != 0
    assert torch.allclose(x.grad[kept], torch.full_like(x.grad[kept], 2.0)) and bool((x.grad[~kept] == 0).all())
