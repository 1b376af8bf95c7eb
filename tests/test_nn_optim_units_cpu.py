"""Unit tests of layers, initialisers, losses, optimizers, schedulers and the loss scaler on the CPU,
one behaviour per test (the topics of the reference's in-module tests under
crates/axonml-nn/src and crates/axonml-optim/src).  Numerics are checked against plain PyTorch."""
import math

import pytest
import torch
import torch.nn.functional as TF

from axonml_b200 import nn, optim
from axonml_b200.nn import functional as F, init


# ------------------------------------------------------------------------------------ parameters
def test_parameter_creation_and_name():
    p = nn.Parameter.new(torch.ones(2, 3))
    assert p.requires_grad and p.shape == (2, 3) and p.name() == ""
    q = nn.Parameter.named("weight", torch.zeros(4), requires_grad=False)
    assert q.name() == "weight" and not q.requires_grad
    q.set_name("bias")
    assert q.name() == "bias" and q.numel_() == 4


def test_parameter_update_and_apply_update():
    p = nn.Parameter.new(torch.ones(3))
    p.update_data(torch.full((3,), 2.0))
    assert p.tolist() == [2.0] * 3
    p.apply_update(torch.ones(3), lr=0.5)
    assert p.tolist() == [1.5] * 3
    p.grad = torch.ones(3)
    p.zero_grad()
    assert p.grad is None or float(p.grad.abs().sum()) == 0


# ----------------------------------------------------------------------------------- initialisers
def test_constant_initialisers():
    assert init.zeros([2, 2]).sum().item() == 0 and init.ones([2, 2]).sum().item() == 4
    assert init.constant([3], 0.25).tolist() == [0.25] * 3 and init.eye(3).equal(torch.eye(3))


def test_uniform_range_stays_in_range():
    u = init.uniform_range([2000], -0.5, 0.25)
    assert -0.5 <= float(u.min()) and float(u.max()) <= 0.25


def test_xavier_and_kaiming_bounds():
    x = init.xavier_uniform(100, 200)
    assert x.shape == (200, 100) and float(x.abs().max()) <= math.sqrt(6 / 300) + 1e-6
    k = init.kaiming_uniform(64, 256)
    assert k.shape == (64, 256) and float(k.abs().max()) <= math.sqrt(6 / 256) + 1e-6
    n = init.kaiming_normal(512, 512)
    assert abs(float(n.std()) - math.sqrt(2 / 512)) < 0.01


def test_orthogonal_rows_are_orthonormal():
    q = init.orthogonal(8, 16)
    assert torch.allclose(q @ q.t(), torch.eye(8), atol=1e-5)
    g = init.orthogonal(4, 4, gain=2.0)
    assert torch.allclose(g @ g.t(), 4 * torch.eye(4), atol=1e-4)


def test_sparse_initialiser_zeroes_the_requested_fraction():
    s = init.sparse(100, 50, 0.9)
    assert s.shape == (100, 50)
    assert 0.85 <= float((s == 0).float().mean()) <= 0.95


def test_init_mode_dispatch():
    assert init.InitMode.Zeros.init([2, 3]).sum().item() == 0
    assert init.InitMode.Constant.init([2], 3.0).tolist() == [3.0, 3.0]
    for mode in init.InitMode:
        assert tuple(mode.init([4, 6]).shape) == (4, 6)


# ------------------------------------------------------------------------------------- functional
def test_functional_activations_match_torch():
    x = torch.randn(5, 7)
    assert torch.allclose(F.relu(x), TF.relu(x)) and torch.allclose(F.sigmoid(x), torch.sigmoid(x), atol=1e-6)
    assert torch.allclose(F.softmax(x, -1), TF.softmax(x, -1), atol=1e-6)
    assert torch.allclose(F.log_softmax(x, -1), TF.log_softmax(x, -1), atol=1e-6)
    assert torch.allclose(F.leaky_relu(x, 0.2), TF.leaky_relu(x, 0.2)) and torch.allclose(F.elu(x), TF.elu(x), atol=1e-6)


def test_functional_dropout_keeps_expectation_and_eval_identity():
    torch.manual_seed(0)
    x = torch.ones(20000)
    y = F.dropout(x, 0.25, training=True)
    assert abs(float(y.mean()) - 1.0) < 0.03 and y.unique().tolist() == pytest.approx([0.0, 1 / 0.75])
    assert F.dropout(x, 0.25, training=False).equal(x)


def test_functional_losses_and_linear():
    a, b = torch.tensor([1.0, 2.0, 3.0]), torch.tensor([1.0, 0.0, 5.0])
    assert F.mse_loss(a, b).item() == pytest.approx(8 / 3)
    logits, y = torch.randn(6, 4), torch.randint(0, 4, (6,))
    assert F.cross_entropy(logits, y).item() == pytest.approx(TF.cross_entropy(logits, y).item(), abs=1e-5)
    p, t = torch.rand(8).clamp(0.05, 0.95), torch.randint(0, 2, (8,)).float()
    assert F.binary_cross_entropy(p, t).item() == pytest.approx(TF.binary_cross_entropy(p, t).item(), abs=1e-5)
    x, w, bias = torch.randn(3, 5), torch.randn(2, 5), torch.randn(2)
    assert torch.allclose(F.linear(x, w, bias), TF.linear(x, w, bias), atol=1e-5)
    assert torch.allclose(F.layer_norm(x, [5]), TF.layer_norm(x, [5]), atol=1e-5)
    assert F.adaptive_avg_pool2d(torch.randn(2, 3, 8, 8), 1).shape == (2, 3, 1, 1)


# ----------------------------------------------------------------------------------------- layers
def test_linear_creation_parameters_and_forward():
    l = nn.Linear(10, 5)
    assert l.weight.shape == (5, 10) and l.bias.shape == (5,) and l.num_parameters() == 55
    assert [n for n, _ in l.named_parameters()] == ["weight", "bias"]
    x = torch.randn(3, 10)
    assert torch.allclose(l(x), x @ l.weight.t() + l.bias, atol=1e-5)
    assert l(torch.randn(2, 4, 10)).shape == (2, 4, 5)


def test_linear_without_bias_and_from_weights():
    l = nn.Linear.with_bias(4, 3, False)
    assert l.bias is None and l.num_parameters() == 12
    w = torch.arange(6.0).reshape(2, 3)
    m = nn.Linear.from_weights(w, torch.tensor([1.0, -1.0]))
    assert m(torch.ones(1, 3)).tolist() == [[4.0, 11.0]]


def test_conv1d_and_conv2d_shapes_match_torch():
    c1 = nn.Conv1d(3, 8, 3, padding=1)
    x1 = torch.randn(2, 3, 20)
    assert torch.allclose(c1(x1), TF.conv1d(x1, c1.weight, c1.bias, padding=1), atol=1e-5)
    c2 = nn.Conv2d.with_options(3, 6, (3, 3), (2, 2), (1, 1), True)
    x2 = torch.randn(2, 3, 9, 9)
    y = c2(x2)
    assert y.shape == (2, 6, 5, 5) and torch.allclose(y, TF.conv2d(x2, c2.weight, c2.bias, 2, 1), atol=1e-5)
    assert c2.weight.shape == (6, 3, 3, 3) and c2.num_parameters() == 6 * 27 + 6


def test_embedding_lookup_batch_and_padding():
    e = nn.Embedding(10, 4, padding_idx=0)
    assert e.weight.shape == (10, 4) and float(e.weight[0].abs().sum()) == 0
    ids = torch.tensor([[1, 2, 0], [3, 3, 9]])
    out = e(ids)
    assert out.shape == (2, 3, 4) and out[0, 0].equal(e.weight[1]) and out[1, 0].equal(out[1, 1])
    out.sum().backward()
    assert float(e.weight.grad[0].abs().sum()) == 0 and float(e.weight.grad[3].sum()) == 8.0
    assert e.lookup(torch.tensor([9])).equal(e.weight[9:10].detach())
    p = nn.Embedding.from_pretrained(torch.eye(3))
    assert p(torch.tensor([2])).tolist() == [[0.0, 0.0, 1.0]]


def test_multihead_attention_self_and_cross():
    torch.manual_seed(0)
    m = nn.MultiHeadAttention(16, 4).eval()
    x, mem = torch.randn(2, 5, 16), torch.randn(2, 7, 16)
    assert m(x).shape == (2, 5, 16) and m.attention(x, mem, mem).shape == (2, 5, 16)
    assert torch.allclose(m(x), m.attention(x, x, x), atol=1e-6)
    assert sum(p.numel() for p in m.parameters()) == 4 * (16 * 16 + 16)
    # causal: the first position sees only itself, so changing later positions leaves it unchanged
    x2 = x.clone()
    x2[:, 1:] += 1.0
    a, b = m.attention(x, x, x, is_causal=True), m.attention(x2, x2, x2, is_causal=True)
    assert torch.allclose(a[:, 0], b[:, 0], atol=1e-5) and not torch.allclose(a[:, 1], b[:, 1], atol=1e-5)


def test_dropout_training_eval_and_zero_probability():
    torch.manual_seed(0)
    d = nn.Dropout(0.5)
    x = torch.ones(4000)
    y = d.train()(x)
    assert 0.4 < float((y == 0).float().mean()) < 0.6 and float(y.max()) == 2.0
    assert d.eval()(x).equal(x) and nn.Dropout(0.0).train()(x).equal(x)


def test_batchnorm_normalises_and_tracks_running_statistics():
    torch.manual_seed(0)
    b = nn.BatchNorm1d(4)
    x = torch.randn(64, 4) * 3 + 5
    y = b.train()(x)
    assert torch.allclose(y.mean(0), torch.zeros(4), atol=1e-4) and torch.allclose(y.var(0, unbiased=False), torch.ones(4), atol=1e-2)
    assert torch.allclose(b.running_mean, 0.1 * x.mean(0), atol=1e-4)
    z = b.eval()(x)
    assert not torch.allclose(z, y)
    b2 = nn.BatchNorm2d(3)
    ref = torch.nn.BatchNorm2d(3)
    x2 = torch.randn(4, 3, 5, 5)
    assert torch.allclose(b2.train()(x2), ref.train()(x2), atol=1e-4)
    assert [n for n, _ in b2.named_parameters()] == ["weight", "bias"]


def test_layernorm_groupnorm_instancenorm_match_torch():
    x = torch.randn(3, 6, 4, 4)
    g = nn.GroupNorm(2, 6)
    assert torch.allclose(g(x), TF.group_norm(x, 2, g.weight, g.bias), atol=1e-4)
    inorm = nn.InstanceNorm2d(6)
    assert torch.allclose(inorm(x), TF.instance_norm(x), atol=1e-4)
    ia = nn.InstanceNorm2d.with_affine(6)
    assert ia.weight.shape == (6,) and torch.allclose(ia(x), TF.instance_norm(x), atol=1e-4)
    ln = nn.LayerNorm(8)
    v = torch.randn(5, 8)
    y = ln(v)
    assert torch.allclose(y.mean(-1), torch.zeros(5), atol=1e-5) and torch.allclose(y, TF.layer_norm(v, [8]), atol=1e-5)
    r = nn.RMSNorm(8)
    assert torch.allclose(r(v), v / (v.pow(2).mean(-1, keepdim=True) + r.eps).sqrt(), atol=1e-5)


def test_pooling_layers_values():
    x = torch.arange(16.0).reshape(1, 1, 4, 4)
    assert nn.MaxPool2d(2)(x).flatten().tolist() == [5, 7, 13, 15]
    assert nn.AvgPool2d(2)(x).flatten().tolist() == [2.5, 4.5, 10.5, 12.5]
    assert nn.AdaptiveAvgPool2d(1)(x).item() == 7.5 and nn.AdaptiveAvgPool2d((2, 2))(x).shape == (1, 1, 2, 2)
    assert nn.MaxPool1d(2)(torch.tensor([[[1.0, 3.0, 2.0, 0.0]]])).flatten().tolist() == [3.0, 2.0]
    assert nn.AvgPool1d(2)(torch.tensor([[[1.0, 3.0, 2.0, 0.0]]])).flatten().tolist() == [2.0, 1.0]


@pytest.mark.parametrize("kind", ["RNN", "LSTM", "GRU"])
def test_recurrent_layers_shapes_and_gradients(kind):
    torch.manual_seed(0)
    m = getattr(nn, kind)(6, 8, num_layers=2)
    x = torch.randn(3, 5, 6, requires_grad=True)
    out = m(x)
    seq = out[0] if isinstance(out, tuple) else out
    assert seq.shape == (3, 5, 8) and m.forward_last(x).shape == (3, 8) and m.forward_mean(x).shape == (3, 8)
    seq.sum().backward()
    assert x.grad is not None and all(p.grad is not None for p in m.parameters())


def test_rnn_cell_single_step_formula():
    c = nn.RNNCell(3, 4)
    x, h = torch.randn(2, 3), torch.randn(2, 4)
    out = c(x, h)
    names = dict(c.named_parameters())
    w_ih = next(v for k, v in names.items() if "ih" in k and v.dim() == 2)
    w_hh = next(v for k, v in names.items() if "hh" in k and v.dim() == 2)
    b = sum(v for k, v in names.items() if v.dim() == 1)
    assert torch.allclose(out, torch.tanh(x @ w_ih.t() + h @ w_hh.t() + b), atol=1e-5)


def test_sequential_construction_forward_and_names():
    s = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 2))
    assert s.len() == 3 and not s.is_empty() and s(torch.randn(5, 4)).shape == (5, 2)
    assert s.num_parameters() == 4 * 8 + 8 + 8 * 2 + 2
    n = nn.Sequential.new().add_named("fc", nn.Linear(2, 2)).add(nn.Sigmoid())
    assert [k for k, _ in n.named_parameters()] == ["fc.weight", "fc.bias"]
    assert float(n(torch.zeros(1, 2)).min()) > 0


def test_module_list_holds_and_iterates_modules():
    ml = nn.ModuleList([nn.Linear(3, 3) for _ in range(3)])
    assert ml.len() == 3 and len(list(ml.iter())) == 3 and not ml.is_empty()
    ml.push(nn.Linear(3, 1))
    x = torch.randn(2, 3)
    for layer in ml:
        x = layer(x)
    assert x.shape == (2, 1) and ml.get(3).weight.shape == (1, 3) and len(list(ml.parameters())) == 8


def test_module_train_eval_and_state_dict_round_trip():
    a, b = nn.Sequential(nn.Linear(3, 4), nn.BatchNorm1d(4)), nn.Sequential(nn.Linear(3, 4), nn.BatchNorm1d(4))
    assert a.is_training() and not a.eval().is_training() and a.set_training(True).is_training()
    a(torch.randn(8, 3))
    b.load_state_dict(a.state_dict())
    x = torch.randn(5, 3)
    assert torch.allclose(a.eval()(x), b.eval()(x))
    assert "1.running_mean" in a.state_dict()


def test_activation_modules():
    x = torch.tensor([-1.0, 0.0, 2.0])
    assert nn.ReLU()(x).tolist() == [0, 0, 2] and nn.Identity()(x).equal(x)
    assert nn.LeakyReLU(0.1)(x).tolist() == pytest.approx([-0.1, 0, 2])
    assert torch.allclose(nn.Sigmoid()(x), torch.sigmoid(x)) and torch.allclose(nn.Tanh()(x), torch.tanh(x))
    assert torch.allclose(nn.Softmax(-1)(x).sum(), torch.tensor(1.0)) and torch.allclose(nn.LogSoftmax(-1)(x).exp().sum(), torch.tensor(1.0))
    assert torch.allclose(nn.SiLU()(x), TF.silu(x), atol=1e-6) and torch.allclose(nn.ELU()(x), TF.elu(x), atol=1e-6)


# ----------------------------------------------------------------------------------------- losses
def test_mse_loss_zero_and_nonzero_with_reductions():
    a = torch.tensor([1.0, 2.0])
    assert nn.MSELoss()(a, a).item() == 0
    b = torch.tensor([2.0, 4.0])
    assert nn.MSELoss()(a, b).item() == 2.5 and nn.MSELoss(nn.Reduction.Sum)(a, b).item() == 5.0
    assert nn.MSELoss.with_reduction(nn.Reduction.None_ if hasattr(nn.Reduction, "None_") else list(nn.Reduction)[0])(a, b).numel() in (1, 2)
    assert nn.L1Loss()(a, b).item() == 1.5


def test_cross_entropy_matches_torch_and_honours_ignore_index():
    logits, y = torch.randn(8, 5), torch.tensor([0, 1, 2, 3, 4, -100, 1, 2])
    ours, ref = nn.CrossEntropyLoss()(logits, y), TF.cross_entropy(logits, y, ignore_index=-100)
    assert ours.item() == pytest.approx(ref.item(), abs=1e-5)
    lp = TF.log_softmax(logits, -1)
    assert nn.NLLLoss()(lp[:5], y[:5]).item() == pytest.approx(TF.nll_loss(lp[:5], y[:5]).item(), abs=1e-5)


def test_bce_and_smooth_l1_losses():
    p, t = torch.tensor([0.9, 0.2]), torch.tensor([1.0, 0.0])
    assert nn.BCELoss()(p, t).item() == pytest.approx(-(math.log(0.9) + math.log(0.8)) / 2, abs=1e-6)
    z = torch.tensor([2.0, -1.0])
    assert nn.BCEWithLogitsLoss()(z, t).item() == pytest.approx(TF.binary_cross_entropy_with_logits(z, t).item(), abs=1e-6)
    a, b = torch.tensor([0.0, 0.0]), torch.tensor([0.5, 3.0])
    assert nn.SmoothL1Loss()(a, b).item() == pytest.approx((0.125 + 2.5) / 2)
    assert nn.SmoothL1Loss.with_beta(2.0)(a, b).item() == pytest.approx(TF.smooth_l1_loss(a, b, beta=2.0).item())


# -------------------------------------------------------------------------------------- optimizers
def _param(values=(1.0, -2.0)):
    p = nn.Parameter.new(torch.tensor(values))
    p.grad = torch.tensor([0.5, -1.0])
    return p


def test_sgd_plain_step_and_zero_grad():
    p = _param()
    o = optim.SGD([p], lr=0.1)
    o.step()
    assert p.tolist() == pytest.approx([0.95, -1.9])
    o.zero_grad()
    assert p.grad is None or float(p.grad.abs().sum()) == 0
    assert o.get_lr() == 0.1 and o.num_parameters() == 2


def test_sgd_momentum_nesterov_and_weight_decay_match_torch():
    for kw in ({"momentum": 0.9}, {"momentum": 0.9, "nesterov": True}, {"weight_decay": 0.1}, {"momentum": 0.5, "dampening": 0.2}):
        p, q = _param(), torch.nn.Parameter(torch.tensor([1.0, -2.0]))
        o, r = optim.SGD([p], lr=0.1, **kw), torch.optim.SGD([q], lr=0.1, **kw)
        for _ in range(3):
            p.grad, q.grad = torch.tensor([0.5, -1.0]), torch.tensor([0.5, -1.0])
            o.step(), r.step()
        assert torch.allclose(p.detach(), q.detach(), atol=1e-6), kw


def test_sgd_builder_pattern():
    p, q = _param(), torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    o = optim.SGD.new([p], 0.1).momentum(0.8).weight_decay(0.01).nesterov(True)
    r = torch.optim.SGD([q], lr=0.1, momentum=0.8, weight_decay=0.01, nesterov=True)
    for _ in range(2):
        p.grad, q.grad = torch.tensor([0.5, -1.0]), torch.tensor([0.5, -1.0])
        o.step(), r.step()
    assert torch.allclose(p.detach(), q.detach(), atol=1e-6)
    o.set_lr(0.01)
    assert o.get_lr() == 0.01
    assert isinstance(optim.SGD.with_momentum([_param()], 0.1, 0.9), optim.SGD)


@pytest.mark.parametrize("ours,ref,kw", [
    (optim.Adam, torch.optim.Adam, {}), (optim.Adam, torch.optim.Adam, {"weight_decay": 0.1}),
    (optim.Adam, torch.optim.Adam, {"amsgrad": True}), (optim.AdamW, torch.optim.AdamW, {"weight_decay": 0.05}),
    (optim.RMSprop, torch.optim.RMSprop, {}), (optim.RMSprop, torch.optim.RMSprop, {"momentum": 0.9}),
    (optim.RMSprop, torch.optim.RMSprop, {"centered": True})])
def test_adaptive_optimizers_match_torch_over_several_steps(ours, ref, kw):
    torch.manual_seed(0)
    p, q = nn.Parameter.new(torch.tensor([1.0, -2.0, 0.5])), torch.nn.Parameter(torch.tensor([1.0, -2.0, 0.5]))
    o, r = ours([p], lr=0.01, **kw), ref([q], lr=0.01, **kw)
    for _ in range(5):
        g = torch.randn(3)
        p.grad, q.grad = g.clone(), g.clone()
        o.step(), r.step()
    assert torch.allclose(p.detach(), q.detach(), atol=1e-5)


def test_lamb_trust_ratio_scales_the_update():
    p = nn.Parameter.new(torch.full((4,), 2.0))
    p.grad = torch.full((4,), 0.1)
    o = optim.LAMB([p], lr=0.1, weight_decay=0.0)
    o.step()
    # first step: the bias-corrected direction is g/|g| = 1 per element, the trust ratio |w|/|u| = 2
    assert p.tolist() == pytest.approx([2.0 - 0.1 * 2.0] * 4, abs=1e-4)
    z = nn.Parameter.new(torch.zeros(3))
    z.grad = torch.ones(3)
    optim.LAMB([z], lr=0.1).step()
    assert torch.isfinite(z).all() and float(z.abs().sum()) > 0      # zero weight norm -> ratio 1


def test_lamb_weight_decay_enters_the_direction():
    a, b = nn.Parameter.new(torch.tensor([1.0, 2.0])), nn.Parameter.new(torch.tensor([1.0, 2.0]))
    a.grad, b.grad = torch.tensor([0.1, -0.1]), torch.tensor([0.1, -0.1])
    optim.LAMB([a], lr=0.01, weight_decay=0.0).step()
    optim.LAMB([b], lr=0.01, weight_decay=0.5).step()
    assert not torch.allclose(a.detach(), b.detach())


def test_optimizers_reduce_a_quadratic():
    for make in (lambda p: optim.SGD(p, lr=0.1, momentum=0.9), lambda p: optim.Adam(p, lr=0.1),
                 lambda p: optim.RMSprop(p, lr=0.05), lambda p: optim.LAMB(p, lr=0.05)):
        w = nn.Parameter.new(torch.tensor([3.0, -4.0]))
        o = make([w])
        for _ in range(200):
            o.zero_grad()
            (w ** 2).sum().backward()
            o.step()
        assert float((w ** 2).sum()) < 0.05


def test_optimizer_state_dict_round_trip_continues_identically():
    torch.manual_seed(0)
    grads = [torch.randn(3) for _ in range(6)]
    p = nn.Parameter.new(torch.ones(3))
    o = optim.Adam([p], lr=0.05)
    for g in grads[:3]:
        p.grad = g.clone()
        o.step()
    q = nn.Parameter.new(p.detach().clone())
    o2 = optim.Adam([q], lr=0.05)
    o2.load_state_dict(o.state_dict())
    for g in grads[3:]:
        p.grad, q.grad = g.clone(), g.clone()
        o.step(), o2.step()
    assert torch.allclose(p.detach(), q.detach(), atol=1e-7)


def test_param_state_view():
    p = nn.Parameter.new(torch.ones(2))
    p.grad = torch.ones(2)
    o = optim.SGD([p], lr=0.1, momentum=0.9)
    o.step()
    st = o.param_state(p)
    assert st.momentum_buffer is not None and st.momentum_buffer.tolist() == [1.0, 1.0]
    fresh = optim.ParamState.new()
    assert fresh.momentum_buffer is None and fresh.step == 0
    fresh.init_momentum(3)
    assert fresh.momentum_buffer.tolist() == [0.0] * 3


# -------------------------------------------------------------------------------------- schedulers
def _opt(lr=1.0):
    return optim.SGD([nn.Parameter.new(torch.zeros(1))], lr=lr)


def _run(s, o, n):
    out = []
    for _ in range(n):
        s.step()
        out.append(o.get_lr())
    return out


def test_step_lr_and_multi_step_lr():
    o = _opt()
    assert _run(optim.StepLR(o, 2, 0.5), o, 5) == pytest.approx([1.0, 0.5, 0.5, 0.25, 0.25])
    o = _opt()
    assert _run(optim.MultiStepLR(o, [2, 4], 0.1), o, 5) == pytest.approx([1.0, 0.1, 0.1, 0.01, 0.01])


def test_exponential_and_cosine_lr():
    o = _opt()
    assert _run(optim.ExponentialLR(o, 0.5), o, 3) == pytest.approx([0.5, 0.25, 0.125])
    o = _opt()
    lrs = _run(optim.CosineAnnealingLR(o, 10, 0.1), o, 10)
    assert lrs[4] == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.5))) and lrs[-1] == pytest.approx(0.1)
    assert all(a >= b for a, b in zip(lrs, lrs[1:]))


def test_warmup_and_one_cycle_lr():
    o = _opt()
    lrs = _run(optim.WarmupLR(o, 4), o, 6)
    assert lrs[:4] == sorted(lrs[:4]) and lrs[3] == pytest.approx(1.0) and lrs[5] == pytest.approx(1.0)
    o = _opt(0.1)
    s = optim.OneCycleLR(o, max_lr=1.0, total_steps=20, pct_start=0.25)
    lrs = _run(s, o, 20)
    peak = lrs.index(max(lrs))
    assert max(lrs) == pytest.approx(1.0, rel=1e-3) and 3 <= peak <= 5 and lrs[-1] < 1e-3 and lrs[0] < 0.5


def test_reduce_lr_on_plateau_waits_for_patience():
    o = _opt()
    s = optim.ReduceLROnPlateau(o, factor=0.5, patience=2)
    for m in (1.0, 0.9, 0.95, 0.95):
        s.step_with_metric(m)
    assert o.get_lr() == 1.0
    s.step_with_metric(0.95)
    assert o.get_lr() == 0.5
    s2 = optim.ReduceLROnPlateau(_opt(), mode="max", factor=0.1, patience=0, min_lr=0.05)
    s2.step_with_metric(1.0), s2.step_with_metric(0.5), s2.step_with_metric(0.4)
    assert s2.get_last_lr() in (0.05, [0.05])


def test_scheduler_state_dict_round_trip():
    o = _opt()
    s = optim.StepLR(o, 3, 0.1)
    _run(s, o, 4)
    o2 = _opt()
    s2 = optim.StepLR(o2, 3, 0.1)
    s2.load_state_dict(s.state_dict())
    assert s2.get_step() == s.get_step() == 4
    assert _run(s2, o2, 3) == pytest.approx(_run(s, o, 3))


# ------------------------------------------------------------------------------------ loss scaler
def test_grad_scaler_scales_and_unscales():
    s = optim.GradScaler.with_scale(128.0)
    assert s.get_scale() == 128.0 and s.is_enabled()
    assert s.scale_loss(torch.tensor(2.0)).item() == 256.0
    p = nn.Parameter.new(torch.zeros(2))
    p.grad = torch.tensor([128.0, 256.0])
    o = optim.SGD([p], lr=1.0)
    s.unscale_(o)
    assert p.grad.tolist() == [1.0, 2.0] and not s.found_inf()


@pytest.mark.parametrize("bad", [float("inf"), float("nan")])
def test_grad_scaler_skips_the_step_and_backs_off_on_overflow(bad):
    s = optim.GradScaler(init_scale=1024.0, backoff_factor=0.5)
    p = nn.Parameter.new(torch.ones(2))
    p.grad = torch.tensor([1.0, bad])
    o = optim.SGD([p], lr=0.1)
    s.step(o)
    s.update()
    assert p.tolist() == [1.0, 1.0] and s.get_scale() == 512.0


def test_grad_scaler_grows_after_the_interval_and_can_be_disabled():
    s = optim.GradScaler(init_scale=2.0, growth_factor=2.0, growth_interval=3)
    p = nn.Parameter.new(torch.ones(1))
    o = optim.SGD([p], lr=0.0)
    for _ in range(3):
        p.grad = torch.ones(1)
        s.step(o)
        s.update()
    assert s.get_scale() == 4.0
    d = optim.GradScaler(enabled=False)
    assert not d.is_enabled() and d.scale_loss(torch.tensor(3.0)).item() == 3.0
    st = s.state_dict()
    r = optim.GradScaler()
    r.load_state_dict(st)
    assert r.get_scale() == 4.0


def test_clip_grad_norm_and_value():
    p = nn.Parameter.new(torch.zeros(2))
    p.grad = torch.tensor([3.0, 4.0])
    total = optim.clip_grad_norm([p], 1.0)
    assert float(total) == pytest.approx(5.0) and p.grad.norm().item() == pytest.approx(1.0, abs=1e-5)
    p.grad = torch.tensor([3.0, -4.0])
    optim.clip_grad_value([p], 2.0)
    assert p.grad.tolist() == [2.0, -2.0]
