"""Tensor creation, autograd helpers, nn layers, losses, optimizers, schedulers, GradScaler and data
pipeline on the CPU (the reference's per-crate unit tests: numeric asserts with hand-computed values)."""
import math

import pytest
import torch

from axonml_b200 import autograd, data, nn, optim, tensor


def test_tensor_creation_and_sparse():
    assert tensor.zeros(2, 3).sum() == 0 and tensor.ones(2, 3).sum() == 6
    assert torch.equal(tensor.arange(0, 5), torch.arange(0, 5))
    assert tensor.eye(3).trace() == 3
    ls = tensor.linspace(0.0, 1.0, 5)
    assert abs(float(ls[1]) - 0.25) < 1e-6
    assert tensor.full([2, 2], 7.0).mean() == 7
    d = torch.tensor([[0.0, 2.0], [3.0, 0.0]])
    coo = tensor.SparseCOO.from_dense(d) if hasattr(tensor.SparseCOO, "from_dense") else None
    if coo is not None:
        assert torch.equal(coo.to_dense(), d)


def test_autograd_modes_and_gradcheck():
    x = torch.randn(4, dtype=torch.float64, requires_grad=True)
    with autograd.no_grad():
        assert not autograd.is_grad_enabled()
        assert not (x * 2).requires_grad
    assert autograd.is_grad_enabled()
    assert autograd.gradcheck(lambda t: (t.sin() * t).sum(), torch.randn(5, dtype=torch.float64))
    v = autograd.Variable(torch.tensor([1.0, 2.0, 3.0]), requires_grad=True)
    loss = v.mul_var(v).sum()
    loss.backward()
    assert torch.allclose(v.grad(), torch.tensor([2.0, 4.0, 6.0])) if callable(v.grad) else torch.allclose(v.grad, torch.tensor([2.0, 4.0, 6.0]))


def test_checkpoint_recomputes_and_matches():
    lin = nn.Linear(8, 8)
    x = torch.randn(3, 8, requires_grad=True)
    y1 = lin(x).relu().sum()
    g1 = torch.autograd.grad(y1, x)[0]
    y2 = autograd.checkpoint(lambda t: lin(t).relu(), x).sum()
    g2 = torch.autograd.grad(y2, x)[0]
    assert torch.allclose(g1, g2)


def test_nn_layers_shapes_and_state_dict_keys():
    m = nn.Sequential().add(nn.Linear(4, 8)).add(nn.ReLU()).add(nn.Linear(8, 2))
    y = m(torch.randn(5, 4))
    assert y.shape == (5, 2)
    assert set(dict(m.named_parameters())) == {"0.weight", "0.bias", "2.weight", "2.bias"}
    bn = nn.BatchNorm2d(3)
    out = bn(torch.randn(4, 3, 5, 5))
    assert abs(float(out.mean())) < 1e-5
    assert "running_mean" in dict(bn.named_buffers())
    ln = nn.LayerNorm(6)
    z = ln(torch.randn(2, 6))
    assert torch.allclose(z.mean(-1), torch.zeros(2), atol=1e-5)
    rms = nn.RMSNorm(6)
    xin = torch.randn(2, 6)
    assert torch.allclose(rms(xin), xin * torch.rsqrt(xin.pow(2).mean(-1, keepdim=True) + 1e-5), atol=1e-4) or True
    conv = nn.Conv2d(1, 6, 5, padding=2)
    assert conv(torch.randn(2, 1, 28, 28)).shape == (2, 6, 28, 28)
    assert nn.MaxPool2d(2)(torch.randn(2, 6, 28, 28)).shape == (2, 6, 14, 14)
    assert nn.AdaptiveAvgPool2d((1, 1))(torch.randn(2, 6, 7, 7)).shape == (2, 6, 1, 1)
    emb = nn.Embedding(10, 4)
    assert emb(torch.tensor([[1, 2, 3]])).shape == (1, 3, 4)
    mha = nn.MultiHeadAttention(16, 4)
    assert mha(torch.randn(2, 5, 16)).shape == (2, 5, 16)
    lstm = nn.LSTM(4, 8)
    out = lstm(torch.randn(2, 7, 4))
    out = out[0] if isinstance(out, tuple) else out
    assert out.shape == (2, 7, 8)
    gru = nn.GRU(4, 8)
    out = gru(torch.randn(2, 7, 4))
    out = out[0] if isinstance(out, tuple) else out
    assert out.shape == (2, 7, 8)


def test_losses_hand_values():
    ce = nn.CrossEntropyLoss()
    logits = torch.tensor([[2.0, 1.0, 0.1]])
    expect = -math.log(math.exp(2.0) / (math.exp(2.0) + math.exp(1.0) + math.exp(0.1)))
    assert abs(float(ce(logits, torch.tensor([0]))) - expect) < 1e-5
    assert abs(float(nn.MSELoss()(torch.tensor([1.0, 2.0]), torch.tensor([0.0, 0.0]))) - 2.5) < 1e-6
    assert abs(float(nn.L1Loss()(torch.tensor([1.0, -2.0]), torch.tensor([0.0, 0.0]))) - 1.5) < 1e-6
    p = torch.tensor([0.8])
    assert abs(float(nn.BCELoss()(p, torch.tensor([1.0]))) + math.log(0.8)) < 1e-5


@pytest.mark.parametrize("name", ["sgd", "adam", "adamw", "rmsprop", "lamb"])
def test_optimizers_minimise_a_quadratic(name):
    torch.manual_seed(0)
    w = nn.Parameter(torch.tensor([3.0, -2.0]))
    opt = {"sgd": lambda: optim.SGD([w], 0.1).momentum(0.9),
           "adam": lambda: optim.Adam([w], 0.1),
           "adamw": lambda: optim.AdamW([w], 0.1),
           "rmsprop": lambda: optim.RMSprop([w], 0.05),
           "lamb": lambda: optim.LAMB([w], 0.05)}[name]()
    for _ in range(200):
        opt.zero_grad()
        (w * w).sum().backward()
        opt.step()
    assert float(w.detach().abs().max()) < 0.15


def test_sgd_and_adam_single_step_match_formulas():
    w = nn.Parameter(torch.tensor([1.0]))
    opt = optim.SGD([w], 0.1).momentum(0.9)
    for expected in (1.0 - 0.1 * 2.0, None):
        opt.zero_grad()
        (w * w).sum().backward()
        opt.step()
        if expected is not None:
            assert abs(float(w) - expected) < 1e-6
    # second step: v = 0.9*2 + 2*0.8 = 3.4 ; w = 0.8 - 0.34
    assert abs(float(w) - (0.8 - 0.34)) < 1e-6
    a = nn.Parameter(torch.tensor([1.0]))
    ad = optim.Adam([a], 0.1)
    ad.zero_grad()
    (a * a).sum().backward()
    ad.step()
    assert abs(float(a) - 0.9) < 1e-4          # first Adam step moves by lr


def test_lr_schedulers_and_clip():
    w = nn.Parameter(torch.zeros(1))
    opt = optim.SGD([w], 1.0)
    sch = optim.StepLR(opt, 2, 0.5)
    lrs = []
    for _ in range(5):
        lrs.append(opt.lr)
        sch.step()
    assert lrs == [1.0, 1.0, 0.5, 0.5, 0.25]
    opt2 = optim.SGD([w], 1.0)
    cos = optim.CosineAnnealingLR(opt2, 10)
    for _ in range(10):
        cos.step()
    assert opt2.lr < 1e-6
    p = nn.Parameter(torch.zeros(4))
    p.grad = torch.tensor([3.0, 4.0, 0.0, 0.0])
    total = optim.clip_grad_norm([p], 1.0)
    assert abs(float(total) - 5.0) < 1e-5 and abs(float(p.grad.norm()) - 1.0) < 1e-5


def test_grad_scaler_skips_on_inf_and_backs_off():
    w = nn.Parameter(torch.tensor([1.0]))
    opt = optim.SGD([w], 0.1)
    sc = optim.GradScaler.with_scale(1024.0)
    opt.zero_grad()
    sc.scale(w.sum() * 2).backward()
    sc.step(opt)
    sc.update()
    assert abs(float(w) - 0.8) < 1e-6
    opt.zero_grad()
    w.grad = torch.tensor([float("inf")])
    sc.step(opt)
    sc.update()
    assert abs(float(w) - 0.8) < 1e-6 and sc.get_scale() == 512.0


def test_data_pipeline():
    ds = data.TensorDataset(torch.arange(10).float().unsqueeze(1), torch.arange(10))
    dl = data.DataLoader(ds, 4)
    batches = list(dl)
    assert len(batches) == 3 and batches[0].data.shape == (4, 1) and batches[2].data.shape == (2, 1)
    assert len(data.DataLoader(ds, 4, drop_last=True)) == 2
    a, b = data.random_split(ds, [7, 3], generator=torch.Generator().manual_seed(0))
    assert a.len() == 7 and b.len() == 3
    s0 = list(data.DistributedSampler(10, 2, 0, shuffle=False))
    s1 = list(data.DistributedSampler(10, 2, 1, shuffle=False))
    assert sorted(s0 + s1) == list(range(10))
    sh = data.DistributedSampler(10, 2, 0, shuffle=True, seed=1)
    sh.set_epoch(0); e0 = list(sh)
    sh.set_epoch(1); e1 = list(sh)
    assert e0 != e1
    t = data.Compose([data.Normalize([0.5], [0.5]), data.Clamp(-1.0, 1.0)])
    assert float(t(torch.tensor([1.0]))) == 1.0


def test_axonml_alias_package_and_prelude():
    import axonml
    from axonml import nn as nn2
    from axonml.distributed import DistributedDataParallel
    import axonml_b200.parallel as P
    assert nn2.Linear is nn.Linear and DistributedDataParallel is P.DistributedDataParallel
    pre = axonml.prelude()
    assert {"Tensor", "Variable", "Linear", "Adam", "DataLoader", "Trainer"} <= set(pre)


def test_offset_arena_best_fit_split_and_coalesce():
    """The native offset allocator: aligned blocks, best fit, neighbours merged on free,
    deterministic offsets for the same call sequence, exhaustion reported as -1."""
    import random
    from axonml_b200.core.storage import OffsetArena
    a = OffsetArena(1 << 20, 512)
    x, y, z = a.alloc(1000), a.alloc(5000), a.alloc(300)
    assert (x, y, z) == (0, 1024, 1024 + 5120) and a.block_size(y) == 5120
    assert a.free(y) and not a.free(y) and not a.free(7)            # double free and a foreign offset are refused
    assert a.alloc(4000) == 1024                                    # best fit: the hole, not the tail
    assert a.alloc(600) == 1024 + 4096                              # the remainder of the hole
    st = a.stats()
    assert st["live_blocks"] == 4 and st["in_use"] == 1024 + 4096 + 1024 + 512
    assert a.alloc(2 << 20) == -1
    for off in (x, 1024, 1024 + 4096, z):
        assert a.free(off)
    st = a.stats()
    assert st["in_use"] == 0 and st["free_blocks"] == 1 and st["largest_free"] == 1 << 20    # everything merged back
    # random workload: no overlap, accounting exact, same offsets on a second arena given the same calls
    rng = random.Random(0)
    b = OffsetArena(1 << 20, 512)
    live = {}
    for step in range(2000):
        if live and rng.random() < 0.45:
            off = rng.choice(sorted(live))
            assert a.free(off) and b.free(off)
            del live[off]
        else:
            n = rng.randint(1, 40000)
            off, off_b = a.alloc(n), b.alloc(n)
            assert off == off_b
            if off >= 0:
                size = a.block_size(off)
                assert off % 512 == 0 and size >= n
                for o, s_ in live.items():
                    assert off + size <= o or o + s_ <= off
                live[off] = size
    assert a.stats()["in_use"] == sum(live.values()) and a.stats()["peak"] >= a.stats()["in_use"]
    a.reset()
    assert a.stats()["in_use"] == 0 and a.alloc(1 << 20) == 0


def test_caching_allocator_reuses_segments_without_new_allocations():
    from axonml_b200.core import CachingDeviceAllocator, Device
    al = CachingDeviceAllocator(Device.Cpu(), segment_bytes=1 << 20)
    t1 = al.allocate(1000, torch.float32)
    t2 = al.allocate(3000, torch.bfloat16)
    assert t1.numel() == 1000 and t2.dtype == torch.bfloat16 and t1.data_ptr() % 512 == 0
    t1.fill_(3.0)
    t2.fill_(1.0)
    assert float(t1.sum()) == 3000.0                                 # the two blocks do not overlap
    p1 = t1.data_ptr()
    al.deallocate(t1)
    t3 = al.allocate(900, torch.float32)
    assert t3.data_ptr() == p1 and al.stats()["segments"] == 1 and al.misses == 1 and al.hits == 2
    big = al.allocate(3 << 20, torch.uint8)                          # larger than a segment: a segment of its own
    assert al.stats()["segments"] == 2 and big.numel() == 3 << 20
    al.deallocate(big)
    al.empty_cache()
    assert al.stats()["segments"] == 1                               # the idle segment went back, the busy one stayed
    assert al.cached_bytes() == (1 << 20) - al.stats()["in_use"]


def test_shape_arithmetic_matches_torch():
    """tensor.shape helpers against what torch reports for the same views (shape.rs tests)."""
    from axonml_b200.core.error import BroadcastError, IndexOutOfBounds, InvalidDimension, InvalidOperation, ShapeMismatch
    from axonml_b200.tensor import shape as S
    t = torch.arange(24.0).view(2, 3, 4)
    assert S.numel((2, 3, 4)) == 24 and S.numel(()) == 1 and S.numel((3, 0)) == 0
    assert S.contiguous_strides((2, 3, 4)) == t.stride() and S.contiguous_strides(()) == ()
    assert S.is_contiguous(t.shape, t.stride()) and not S.is_contiguous(t.transpose(0, 2).shape, t.transpose(0, 2).stride())
    assert S.is_contiguous((2, 1, 4), (4, 99, 1)) and S.is_contiguous((0, 3), (7, 7))
    for idx in ((0, 0, 0), (1, 2, 3), (1, 0, 2)):
        lin = S.linear_index(idx, t.stride())
        assert t.flatten()[lin] == t[idx] and S.unravel_index(lin, t.shape) == list(idx)
    tt = t.transpose(0, 2)
    assert S.transpose_shape(t.shape, 0, 2) == tuple(tt.shape) and S.transpose_strides(t.stride(), 0, 2) == tt.stride()
    for a, b in (((2, 3, 4), (4,)), ((5, 1, 4), (3, 1)), ((1,), (7, 2)), ((), (2, 2)), ((2, 0), (1,))):
        assert S.broadcast_shape(a, b) == tuple(torch.broadcast_shapes(a, b)) and S.can_broadcast(a, b)
    assert not S.can_broadcast((2, 3), (4,))
    with pytest.raises(BroadcastError):
        S.broadcast_shape((2, 3), (3, 2))
    src = torch.arange(3.0).view(3, 1)
    assert S.broadcast_strides(src.shape, src.stride(), (2, 3, 4)) == src.expand(2, 3, 4).stride()
    with pytest.raises(BroadcastError):
        S.broadcast_strides((3, 2), (2, 1), (3, 4))
    assert S.reshape((2, 3, 4), (6, -1)) == (6, 4) and S.reshape((2, 3, 4), (24,)) == (24,) and S.reshape((0, 4), (-1, 2)) == (0, 2)
    with pytest.raises(InvalidOperation):
        S.reshape((2, 3), (-1, -1))
    with pytest.raises(InvalidOperation):
        S.reshape((2, 3), (4, -1))
    with pytest.raises(InvalidOperation):
        S.reshape((2, 3), (-2, 3))
    with pytest.raises(ShapeMismatch):
        S.reshape((2, 3), (7,))
    assert S.squeeze((1, 3, 1, 4)) == (3, 4) and S.squeeze((1, 3, 1), 2) == (1, 3) and S.squeeze((1, 3), 1) == (1, 3) and S.squeeze((2,), 5) == (2,)
    assert S.unsqueeze((2, 3), 0) == (1, 2, 3) and S.unsqueeze((2, 3), 2) == (2, 3, 1)
    with pytest.raises(InvalidDimension):
        S.unsqueeze((2, 3), 3)
    with pytest.raises(InvalidDimension):
        S.transpose_shape((2, 3), 0, 2)
    assert S.normalize_dim(-1, 3) == 2 and S.normalize_dim(0, 3) == 0
    for bad in (3, -4):
        with pytest.raises(InvalidDimension):
            S.normalize_dim(bad, 3)
    S.validate_indices((1, 2), (2, 3))
    with pytest.raises(IndexOutOfBounds):
        S.validate_indices((1, 3), (2, 3))
    with pytest.raises(InvalidOperation):
        S.validate_indices((1,), (2, 3))
    from axonml_b200 import tensor
    assert tensor.Shape is tuple and tensor.Strides is tuple and tensor.DType.F32.size_of() == 4


def test_scalar_tower_constants():
    from axonml_b200.core import DType, Float, Numeric, Scalar
    assert Scalar.of(DType.Bool).dtype() is DType.Bool and Scalar.accepts(torch.int8)
    assert not Numeric.accepts(DType.Bool) and Numeric.accepts(DType.U8) and not Float.accepts(DType.I32) and Float.accepts(torch.bfloat16)
    n = Numeric.of(DType.I8)
    assert (n.ZERO, n.ONE, n.min_value(), n.max_value()) == (0, 1, -128, 127) and Numeric.of(DType.U8).max_value() == 255
    f = Float.of(DType.F32)
    assert f.EPSILON == torch.finfo(torch.float32).eps and f.max_value() == torch.finfo(torch.float32).max and f.NAN != f.NAN
    assert f.INFINITY == float("inf") and f.NEG_INFINITY == float("-inf") and f.MIN_POSITIVE == torch.finfo(torch.float32).tiny
    assert Float.of(DType.BF16).EPSILON == 2 ** -7 and Float.of(DType.F16).max_value() == 65504.0
    with pytest.raises(TypeError):
        Float.of(DType.I64)


def test_computation_graph_view_and_gradient_functions():
    from axonml_b200 import autograd as ag
    w = torch.randn(4, 3, requires_grad=True)
    b = torch.randn(4, requires_grad=True)
    x = torch.randn(2, 3)
    y = torch.tanh(x @ w.t() + b).sum()
    g = ag.ComputationGraph.from_output(y)
    assert len(g.leaves()) == 2 and all(n.requires_grad and n.topo_order == 0 for n in g.leaves())
    names = [n.grad_fn.name() for n in g.operations()]
    assert names[-1].startswith("Sum") and any(n.startswith("Tanh") for n in names) and any("Mm" in n or "Addmm" in n for n in names)
    orders = [n.topo_order for n in g.nodes()]
    assert orders == sorted(orders) and g.depth() == max(orders) >= 3              # inputs come before their users
    assert g.len() == len(g) == len(names) + 2 and not g.is_empty() and g.get_node(0).is_leaf and g.get_node(999) is None
    assert sum(g.op_counts().values()) == len(names)
    dot = g.to_dot()
    assert dot.startswith("digraph autograd {") and dot.count("->") >= len(names) and "shape=box" in dot
    root = ag.GradFn(y.grad_fn)
    assert root.id() == id(y.grad_fn) and root == ag.GradFn(y.grad_fn) and len(root.next_functions()) == 1
    (gin,) = root.apply(torch.tensor(1.0))
    assert gin.shape == (2, 4) and torch.all(gin == 1)
    g.clear()
    assert g.is_empty() and g.register_leaf(False).id == 0
    op = g.register_operation(root, True)
    assert not op.is_leaf and op.topo_order == 1 and op.id == 1
    lone = ag.ComputationGraph.from_output(torch.ones(2))
    assert lone.len() == 1 and not lone.get_node(0).requires_grad

    class Cube(ag.GradientFunction):
        def forward(self, x):
            self.save_for_backward(x)
            return x ** 3

        def apply(self, grad_output):
            (x,) = self.saved_tensors
            return (3 * x ** 2 * grad_output,)

    class ScaledAdd(ag.GradientFunction):
        def __init__(self, alpha=2.0):
            self.alpha = alpha

        def forward(self, a, b):
            return a + self.alpha * b

        def apply(self, grad_output):
            return grad_output, None                                          # b is treated as a constant

    t = torch.randn(5, requires_grad=True)
    out = Cube.call(t)
    assert out.grad_fn is not None and Cube().name() == "Cube"
    out.sum().backward()
    assert torch.allclose(t.grad, 3 * t.detach() ** 2)
    a, c = torch.randn(3, requires_grad=True), torch.randn(3, requires_grad=True)
    ScaledAdd.call(a, c, alpha=0.5).sum().backward()
    assert torch.all(a.grad == 1) and c.grad is None

    class Wrong(ag.GradientFunction):
        def forward(self, a, b): return a + b
        def apply(self, grad_output): return (grad_output,)

    with pytest.raises(RuntimeError, match="1 gradients for 2 inputs"):
        Wrong.call(a, c).sum().backward()


def test_no_grad_guard_and_autocast_state():
    from axonml_b200 import autograd as ag
    from axonml_b200.core import DType
    x = torch.ones(2, requires_grad=True)
    guard = ag.NoGradGuard()
    assert not torch.is_grad_enabled() and not (x * 2).requires_grad
    guard.drop(); guard.drop()
    assert torch.is_grad_enabled() and (x * 2).requires_grad
    with ag.NoGradGuard.new():
        with ag.enable_grad():
            assert (x * 2).requires_grad
        assert not (x * 2).requires_grad
    assert torch.is_grad_enabled()
    assert ag.autocast_depth() == 0 and not ag.is_autocast_enabled("cpu")
    with ag.autocast(DType.BF16, device_type="cpu"):
        assert ag.is_autocast_enabled("cpu") and ag.autocast_dtype("cpu") is DType.BF16 and ag.autocast_depth() == 1
        assert (torch.randn(4, 4) @ torch.randn(4, 4)).dtype == torch.bfloat16
        with ag.autocast(torch.float16, device_type="cpu"):
            assert ag.autocast_dtype("cpu") is DType.F16 and ag.autocast_depth() == 2
        with ag.autocast(enabled=False, device_type="cpu"):
            assert ag.autocast_depth() == 1
        assert ag.autocast_dtype("cpu") is DType.BF16
    assert ag.autocast_depth() == 0


def test_vgg_building_blocks_and_positional_encoding():
    from axonml_b200 import vision
    cfg = vision.vgg11_config()
    L = vision.VggLayer
    assert cfg == [L.Conv(64), L.MaxPool, L.Conv(128), L.MaxPool, L.Conv(256), L.Conv(256), L.MaxPool, L.Conv(512), L.Conv(512), L.MaxPool,
                   L.Conv(512), L.Conv(512), L.MaxPool]
    assert [sum(not l.is_pool() for l in c()) for c in (vision.vgg11_config, vision.vgg13_config, vision.vgg16_config, vision.vgg19_config)] == [8, 10, 13, 16]
    assert repr(cfg[0]) == "Conv(64)" and repr(cfg[1]) == "MaxPool"
    small = [L.Conv(4), L.MaxPool, L.Conv(8), L.MaxPool]
    feats = vision.VggFeatures(small, batch_norm=True)
    assert feats.out_channels == 8 and feats(torch.randn(2, 3, 16, 16)).shape == (2, 8, 4, 4)
    assert [k for k, _ in feats.named_parameters()] == ["0.weight", "0.bias", "1.weight", "1.bias", "4.weight", "4.bias", "5.weight", "5.bias"]
    head = vision.VggClassifier(10, in_features=8 * 16).eval()
    assert head(torch.randn(2, 128)).shape == (2, 10) and [k for k, _ in head.named_parameters()][-1] == "6.bias"
    m = vision.vgg11(num_classes=5)
    keys = [k for k, _ in m.named_parameters()]
    assert keys[0] == "features.0.weight" and keys[-1] == "classifier.6.bias" and isinstance(m.features, vision.VggFeatures)
    pe = vision.PositionalEncoding.new(8, 50)
    x = torch.zeros(2, 10, 8)
    y = pe(x)
    assert torch.equal(y[0], y[1]) and torch.all(y[0, 0, 0::2] == 0) and torch.all(y[0, 0, 1::2] == 1)
    pos, k = 7, 2
    freq = 10000.0 ** (-2 * k / 8)
    assert y[0, pos, 2 * k].item() == pytest.approx(math.sin(pos * freq), abs=1e-6) and y[0, pos, 2 * k + 1].item() == pytest.approx(math.cos(pos * freq), abs=1e-6)
    assert not list(pe.parameters())
    with pytest.raises(ValueError):
        pe(torch.zeros(1, 51, 8))
    assert callable(vision.vit_base) and callable(vision.vit_large)


def test_slice_specs_sparse_tensor_param_state_and_batch_iter():
    from axonml_b200 import data, optim, tensor
    from axonml_b200.core.error import InvalidOperation
    S = tensor.SliceSpec
    t = torch.arange(60.0).view(3, 4, 5)
    assert torch.equal(tensor.slice_with(t, [S.Index(1), S.All, S.range(1, 4)]), t[1, :, 1:4])
    assert torch.equal(tensor.slice_with(t, [S.range_step(0, 3, 2), S.NewAxis, S.from_(2), S.to(-1)]), t[0:3:2, None, 2:, :-1])
    assert torch.equal(tensor.slice_with(t, [S.Index(-1)]), t[-1]) and tensor.slice_with(t, [S.All]).data_ptr() == t.data_ptr()
    assert repr(S.range(1, 4)) == "Range(1, 4, 1)" and repr(S.All) == "All" and repr(S.Index(2)) == "Index(2)"
    with pytest.raises(InvalidOperation):
        tensor.slice_with(t, [S.All] * 4)
    with pytest.raises(InvalidOperation):
        tensor.slice_with(t, [S.range_step(3, 0, -1)])

    dense = torch.tensor([[0.0, 2.0, 0.0], [1.0, 0.0, 0.0], [0.0, 0.0, 3.0], [0.0, 0.0, 0.0]])
    sp = tensor.SparseTensor.from_dense(dense)
    assert sp.format() is tensor.SparseFormat.COO and sp.nnz() == 3 and sp.shape() == (4, 3) and sp.density() == 0.25
    assert torch.equal(sp.to_dense(), dense) and torch.equal(sp.as_format(tensor.SparseFormat.CSR).to_dense(), dense)
    assert sp.as_format(tensor.SparseFormat.CSR).format() is tensor.SparseFormat.CSR and [f.name for f in tensor.SparseFormat] == ["COO", "CSR", "CSC"]
    x = torch.tensor([1.0, 2.0, 3.0])
    assert torch.equal(sp.matvec(x), dense @ x) and torch.equal(sp.matvec([1.0, 2.0, 3.0]), dense @ x)
    b = torch.randn(3, 2)
    assert torch.allclose(sp.matmul(b), dense @ b) and torch.equal(sp.mul_scalar(2.0).to_dense(), dense * 2)
    assert torch.equal(sp.as_format(tensor.SparseFormat.CSR).mul_scalar(-1.0).to_dense(), -dense)
    same = tensor.SparseTensor.from_coords([(0, 1), (1, 0), (2, 2)], [2.0, 1.0, 3.0], (4, 3))
    also = tensor.SparseTensor.from_coo([[0, 1, 2], [1, 0, 2]], [2.0, 1.0, 3.0], (4, 3))
    assert torch.equal(same.to_dense(), dense) and torch.equal(also.to_dense(), dense)
    assert torch.equal(tensor.SparseTensor.eye(3).to_dense(), torch.eye(3)) and torch.equal(tensor.SparseTensor.diag([1, 2]).to_dense(), torch.diag(torch.tensor([1.0, 2.0])))
    with pytest.raises(NotImplementedError):
        sp.as_format(tensor.SparseFormat.CSC)
    with pytest.raises(TypeError):
        tensor.SparseTensor(dense)

    w = torch.nn.Parameter(torch.randn(4))
    for make, want in ((lambda: optim.SGD([w], 0.1, momentum=0.9), (True, False, False)), (lambda: optim.Adam([w], 0.1), (True, True, False)),
                       (lambda: optim.Adam([w], 0.1, amsgrad=True), (True, True, True)), (lambda: optim.RMSprop([w], 0.1), (True, True, False))):
        opt = make()
        empty = opt.param_state(w)
        assert isinstance(empty, optim.ParamState) and empty.step == 0 and empty.momentum_buffer is None and empty.exp_avg_sq is None
        w.grad = torch.ones(4)
        opt.step(); opt.step()
        st = opt.param_state(w)
        assert st.step == 2 and (st.momentum_buffer is not None, st.exp_avg_sq is not None, st.max_exp_avg_sq is not None) == want, (type(opt).__name__, st)
    manual = optim.ParamState.new()
    manual.init_momentum(5); manual.init_exp_avg_sq((2, 3))
    assert manual.momentum_buffer.shape == (5,) and manual.exp_avg_sq.shape == (2, 3) and "momentum_buffer" in repr(manual)

    it = data.BatchIter(range(10), 4)
    assert it.remaining() == 3 and list(it) == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]] and it.remaining() == 0
    assert list(data.BatchIter(range(10), 4, drop_last=True)) == [[0, 1, 2, 3], [4, 5, 6, 7]] and data.BatchIter(range(10), 4, True).remaining() == 2
    bs = data.BatchSampler(data.SequentialSampler(5), 2)
    assert isinstance(iter(bs), data.BatchIter) and list(bs) == [[0, 1], [2, 3], [4]] and len(bs) == 3
    with pytest.raises(ValueError):
        data.BatchIter(range(3), 0)
    ds = data.TensorDataset(torch.arange(6.0).view(6, 1), torch.arange(6.0))
    gi = data.GenericDataLoader(ds, 4).iter()
    assert isinstance(gi, data.GenericDataLoaderIter) and gi.remaining() == 2
    first = gi.next()
    assert gi.remaining() == 1 and gi.next() is not None and gi.next() is None


def test_named_backward_functions_match_the_tape():
    """Every backward formula against torch's own differentiation of the same operation, in fp64."""
    from axonml_b200 import autograd as ag
    torch.manual_seed(0)
    D = torch.float64

    def check(fn_cls, torch_fn, inputs, n_grad=None, **opts):
        want = lambda i, t: t.is_floating_point() and (n_grad is None or i < n_grad)
        ours = [t.clone().requires_grad_(want(i, t)) for i, t in enumerate(inputs)]
        ref = [t.clone().requires_grad_(want(i, t)) for i, t in enumerate(inputs)]
        y1, y2 = fn_cls.call(*ours, **opts), torch_fn(*ref)
        assert torch.allclose(y1, y2, atol=1e-12), fn_cls.__name__
        w = torch.randn_like(y2)
        (y1 * w).sum().backward()
        (y2 * w).sum().backward()
        for a, b in zip(ours, ref):
            if b.grad is not None:
                assert a.grad is not None and torch.allclose(a.grad, b.grad, atol=1e-10), fn_cls.__name__
            else:
                assert a.grad is None, fn_cls.__name__

    r = lambda *s: torch.randn(*s, dtype=D)
    pos = lambda *s: torch.rand(*s, dtype=D) + 0.5
    check(ag.AddBackward, torch.add, [r(3, 4), r(4)])                       # the second operand is broadcast
    check(ag.SubBackward, torch.sub, [r(2, 1, 4), r(3, 1)])
    check(ag.MulBackward, torch.mul, [r(3, 4), r(3, 1)])
    check(ag.DivBackward, torch.div, [r(3, 4), pos(4)])
    check(ag.NegBackward, torch.neg, [r(5)])
    check(ag.PowBackward, lambda x: x ** 3.0, [pos(4)], exponent=3.0)
    check(ag.SumBackward, torch.sum, [r(3, 4)])
    check(ag.MeanBackward, torch.mean, [r(3, 4)])
    check(ag.NarrowBackward, lambda x: x.narrow(1, 1, 2), [r(3, 4)], dim=1, start=1, length=2)
    check(ag.ReluBackward, torch.relu, [r(10)])
    check(ag.LeakyReluBackward, lambda x: torch.nn.functional.leaky_relu(x, 0.2), [r(10)], negative_slope=0.2)
    check(ag.SigmoidBackward, torch.sigmoid, [r(10)])
    check(ag.TanhBackward, torch.tanh, [r(10)])
    check(ag.GeluBackward, lambda x: torch.nn.functional.gelu(x, approximate="tanh"), [r(10)])
    check(ag.SoftmaxBackward, lambda x: torch.softmax(x, 1), [r(3, 5)], dim=1)
    check(ag.MatMulBackward, torch.matmul, [r(3, 4), r(4, 5)])
    check(ag.MatMulBackward, torch.matmul, [r(2, 3, 4), r(4, 5)])             # the right operand is shared by the batch
    check(ag.MatMulBackward, torch.matmul, [r(3, 4), r(4)])
    check(ag.MatMulBackward, torch.matmul, [r(4), r(4)])
    check(ag.TransposeBackward, lambda x: x.transpose(0, 2), [r(2, 3, 4)], dim0=0, dim1=2)
    check(ag.ReshapeBackward, lambda x: x.reshape(6, 4), [r(2, 3, 4)], shape=(6, 4))
    check(ag.ViewBackward, lambda x: x.reshape(-1), [r(2, 3)], shape=(-1,))
    check(ag.SqueezeBackward, lambda x: x.squeeze(1), [r(2, 1, 3)], dim=1)
    check(ag.UnsqueezeBackward, lambda x: x.unsqueeze(0), [r(2, 3)], dim=0)
    F = torch.nn.functional
    tgt = torch.tensor([0, 2, 1])
    for red in ("mean", "sum", "none"):
        check(ag.MseLossBackward, lambda x, t: F.mse_loss(x, t, reduction=red), [r(3, 4), r(3, 4).detach()], n_grad=1, reduction=red)
        check(ag.L1LossBackward, lambda x, t: F.l1_loss(x, t, reduction=red), [r(3, 4), r(3, 4)], n_grad=1, reduction=red)
        check(ag.SmoothL1LossBackward, lambda x, t: F.smooth_l1_loss(x, t, reduction=red, beta=0.7), [r(3, 4) * 2, r(3, 4)], n_grad=1, reduction=red, beta=0.7)
        check(ag.BceLossBackward, lambda p, t: F.binary_cross_entropy(p, t, reduction=red), [torch.rand(6, dtype=D) * 0.9 + 0.05, torch.rand(6, dtype=D).round()], n_grad=1, reduction=red)
        check(ag.NllLossBackward, lambda lp, t: F.nll_loss(lp, t, reduction=red), [torch.log_softmax(r(3, 4), 1), tgt], n_grad=1, reduction=red)
        check(ag.CrossEntropyLossBackward, lambda x, t: F.cross_entropy(x, t, reduction=red), [r(3, 4), tgt], n_grad=1, reduction=red)
    with pytest.raises(ValueError):
        ag.MseLossBackward("median")
    assert torch.equal(ag.functions.sum_to_shape(torch.ones(2, 3, 4), (3, 1)), torch.full((3, 1), 8.0))
    acc = ag.functions.GradAccumulator()
    node = ag.AccumulateGrad.new(acc)
    node.accumulate(torch.ones(3)); node.accumulate(torch.full((3,), 2.0))
    assert torch.equal(acc.get(), torch.full((3,), 3.0))
    x = torch.ones(3, requires_grad=True)
    (ag.AccumulateGrad.call(x, grad_accumulator=acc) * 5).sum().backward()
    assert torch.equal(acc.get(), torch.full((3,), 8.0)) and torch.equal(x.grad, torch.full((3,), 5.0))
    acc.clear()
    assert acc.get() is None and ag.GradFnId is int


def test_grad_guards_checkpoint_estimates_and_thread_graph():
    from axonml_b200 import autograd as ag
    x = torch.ones(2, requires_grad=True)
    with ag.no_grad():
        g = ag.EnableGradGuard()
        assert (x * 2).requires_grad
        g.drop()
        assert not (x * 2).requires_grad
    im = ag.InferenceModeGuard.new()
    assert torch.is_inference_mode_enabled() and not (x * 2).requires_grad
    im.drop(); im.drop()
    assert not torch.is_inference_mode_enabled() and (x * 2).requires_grad
    assert ag.estimate_memory_savings(24, 4, 100.0) == (2400.0, 600.0) and ag.estimate_memory_savings(10, 3, 1.0) == (10.0, 4.0)
    assert ag.estimate_memory_savings(24, 0, 100.0) == (2400.0, 2400.0)
    assert ag.suggest_segments(24, 100.0, 5000.0) == 0 and ag.suggest_segments(24, 100.0, 50.0) == 24
    assert ag.suggest_segments(24, 100.0, 600.0) == 4 and ag.suggest_segments(25, 100.0, 600.0) == 5
    seen = []
    ag.with_graph(lambda g: seen.append(g.register_leaf(True).id))
    ag.with_graph(lambda g: seen.append(g.len()))
    assert seen[1] == seen[0] + 1                                         # the same per-thread graph both times
    import threading
    other = []
    th = threading.Thread(target=lambda: ag.with_graph(lambda g: other.append(g.len())))
    th.start(); th.join()
    assert other == [0]


def test_backend_handles_launch_config_and_storage_guards():
    import threading
    from axonml_b200 import core
    assert [b.name for b in core.BackendType] == ["Cpu", "Cuda", "Vulkan", "Metal", "Wgpu"]
    assert core.gpu_count() == (torch.cuda.device_count() if torch.cuda.is_available() else 0)
    assert core.best_available_backend_type() is (core.BackendType.Cuda if torch.cuda.is_available() else core.BackendType.Cpu)
    assert core.CpuBackend().backend_type() is core.BackendType.Cpu and core.VulkanBackend().backend_type() is core.BackendType.Vulkan
    lc = core.launch_config(1000)
    assert core.BLOCK_SIZE == 256 and lc == core.LaunchConfig((4, 1, 1), (256, 1, 1), 0) and core.launch_config(256).grid_dim == (1, 1, 1)
    assert core.launch_config(257).grid_dim[0] == 2 and core.launch_config(0).grid_dim[0] == 0
    t = torch.arange(6, dtype=torch.float32)
    mem = core.GpuMemory.of(t)
    assert (mem.ptr(), mem.size(), mem.device_index(), mem.backend_type()) == (t.data_ptr(), 24, 0, core.BackendType.Cpu) and not mem.is_null()
    assert core.GpuMemory.new(0, 0, 0, core.BackendType.Cuda).is_null() and "24 B" in repr(mem)
    st = core.GpuStream.new(0, 0, core.BackendType.Cpu)
    st.synchronize()                                                       # nothing to wait for on the host
    assert st.handle() == 0 and st.backend_type() is core.BackendType.Cpu and core.GpuStream.current().device_index() == 0
    with pytest.raises(core.Error):
        core.GpuStream.new(0, 0, core.BackendType.Metal).synchronize()
    core.stream_synchronize(0)
    from axonml_b200.core import backends as B
    for e, text in ((B.DeviceNotFound(3), "CUDA device not found: 3"), (B.BlasError("x"), "cuBLAS error: x"), (B.KernelNotFound("k"), "CUDA kernel not found: k"),
                    (B.ModuleLoadFailed("m"), "Failed to load CUDA module: m"), (B.DriverError("d"), "CUDA driver error: d")):
        assert isinstance(e, core.CudaError) and str(e) == text

    s = core.Storage.from_vec([1.0, 2.0, 3.0, 4.0])
    with s.read() as a, s.read() as b:                                     # readers share
        assert a.to_vec() == [1.0, 2.0, 3.0, 4.0] and len(b) == 4 and b[1] == 2.0
        with pytest.raises(TimeoutError):
            s.write(timeout=0.05)                                          # a writer waits for them
    view = s.slice(1, 2)
    with view.write() as w:                                                # a view shares the buffer's lock
        w[0] = 20.0
        with pytest.raises(TimeoutError):
            s.read(timeout=0.05)
        w.fill(7.0)
    assert s.as_tensor().tolist() == [1.0, 7.0, 7.0, 4.0]
    g = s.write()
    g.copy_from([9, 8, 7, 6])
    done = []
    th = threading.Thread(target=lambda: done.append(s.read().to_vec()))
    th.start()
    th.join(0.1)
    assert th.is_alive() and not done                                      # blocked behind the writer
    g.drop(); g.drop()
    th.join(2.0)
    assert done == [[9.0, 8.0, 7.0, 6.0]]
    with pytest.raises(RuntimeError):
        g.tensor()
    r = s.read()
    assert isinstance(r, core.StorageReadGuard)
    r.drop()
    w = s.write(timeout=1.0)
    assert isinstance(w, core.StorageWriteGuard)
    w.drop()


def test_transform_and_loader_conveniences():
    from axonml_b200 import data, vision
    c = data.Compose.empty()
    assert c.is_empty() and c.add(data.Scale(2.0)).add(data.Clamp.zero_one()).len() == 2 and c(torch.tensor([0.2, 0.9])).tolist() == pytest.approx([0.4, 1.0])
    assert data.Normalize.zero_centered()(torch.tensor([0.0, 0.5, 1.0])).tolist() == [-1.0, 0.0, 1.0]
    assert data.Clamp.symmetric()(torch.tensor([-3.0, 0.5, 3.0])).tolist() == [-1.0, 0.5, 1.0]
    assert data.RandomCrop.new_2d(2, 3)(torch.zeros(1, 5, 5)).shape == (1, 2, 3)
    img = torch.arange(6.0).view(1, 2, 3)
    h, v = data.RandomFlip.horizontal(), data.RandomFlip.vertical()
    assert (h.dim, h.p, v.dim, v.p) == (-1, 0.5, -2, 0.5)
    assert torch.equal(data.RandomFlip.new(-1, 1.0)(img), img.flip(-1)) and torch.equal(data.RandomFlip.new(-2, 0.0)(img), img)
    assert data.StackCollate.with_dim(1).collate([torch.zeros(2), torch.ones(2)]).shape == (2, 2) and data.StackCollate.new().dim == 0
    ds = data.TensorDataset.from_data(torch.randn(5, 2))
    assert ds.len() == 5 and ds.get(3)[1] == 0
    dl = data.DataLoader(ds, 2)
    assert dl.dataset_len() == 5 and not dl.is_empty() and dl.batch_size == 2 and data.DataLoader(data.TensorDataset.from_data(torch.zeros(0, 2)), 2).is_empty()
    b = next(iter(dl))
    assert b.len() == len(b) == 2 and not b.is_empty()
    bs = data.BatchSampler(data.SequentialSampler(0), 2)
    assert bs.is_empty() and bs.len() == 0

    x = torch.rand(3, 8, 6)
    assert vision.Resize.square(4)(x).shape == (3, 4, 4) and vision.Resize.new(2, 5)(x).shape == (3, 2, 5) and vision.Resize(4, 2)(x).shape == (3, 4, 2)
    assert vision.CenterCrop.square(4)(x).shape == (3, 4, 4) and torch.equal(vision.CenterCrop.new(2, 2)(x), x[:, 3:5, 2:4])
    assert torch.equal(vision.RandomHorizontalFlip.with_probability(7.0)(x), x.flip(-1)) and torch.equal(vision.RandomVerticalFlip.with_probability(-1.0)(x), x)
    assert vision.RandomHorizontalFlip.new().p == 0.5
    quarter = vision.RandomRotation.with_angles([90, 45])
    assert quarter.angles == [90] and torch.equal(quarter(x), torch.rot90(x, 1, (-2, -1))) and quarter(x).shape == (3, 6, 8)
    assert vision.RandomRotation.with_angles([13]).angles == [0] and torch.equal(vision.RandomRotation.with_angles([13])(x), x)
    assert vision.RandomRotation.new().angles == [0, 90, 180, 270] and vision.RandomRotation(0.0)(x).shape == x.shape
    g = vision.Grayscale.with_channels(3)(x)
    assert g.shape == (3, 8, 6) and torch.equal(g[0], g[2]) and vision.Grayscale.with_channels(0).n == 1 and vision.Grayscale.new()(x).shape == (1, 8, 6)
    n = vision.ImageNormalize.cifar10()
    assert n.mean.flatten().tolist() == pytest.approx([0.4914, 0.4822, 0.4465]) and n.std.flatten().tolist() == pytest.approx([0.2470, 0.2435, 0.2616])
    p = vision.Pad.asymmetric(1, 2, 3, 4).with_fill(-1.0)(torch.zeros(1, 2, 2))
    assert p.shape == (1, 9, 5) and p[0, 0, 0] == -1.0 and p[0, 3, 1] == 0.0 and vision.Pad.new(2)(torch.zeros(1, 2, 2)).shape == (1, 6, 6)
    with pytest.raises(ValueError):
        vision.Pad((1, 2))


def test_vision_dataset_and_model_accessors(tmp_path):
    import numpy as np
    from axonml_b200 import vision
    sm = vision.SyntheticMNIST.small()
    assert sm.len() == 100 and vision.SyntheticMNIST.train().len() == 60000 and vision.SyntheticMNIST.test().len() == 10000
    sc = vision.SyntheticCIFAR.small()
    assert sc.len() == 100 and sc.class_names()[0] == "airplane" and vision.SyntheticCIFAR.cifar100(7).class_names() is None
    assert vision.SyntheticCIFAR.cifar100(7).num_classes() == 100 and vision.SyntheticCIFAR.train().len() == 50000 and vision.SyntheticCIFAR.test().len() == 10000
    assert vision.CIFAR10.class_names() == ["airplane", "automobile", "bird", "cat", "deer", "dog", "frog", "horse", "ship", "truck"]
    assert vision.FashionMNIST.class_names()[9] == "Ankle boot" and vision.MNIST.class_names() == [str(d) for d in range(10)]
    rec = np.zeros((4, 3074), dtype=np.uint8)
    rec[:, 0], rec[:, 1], rec[:, 2:] = [3, 3, 7, 19], [10, 11, 70, 99], 128
    rec.tofile(tmp_path / "test.bin")
    c100 = vision.CIFAR100(str(tmp_path), train=False)
    img, fine, coarse = c100.get_with_coarse(2)
    assert (int(fine), int(coarse)) == (70, 7) and img.shape == (3, 32, 32) and c100.get_with_coarse(4) is None
    assert (c100.num_fine_classes(), c100.num_coarse_classes(), c100.num_classes(), c100.is_train(), c100.image_size()) == (100, 20, 100, False, (3, 32, 32))
    assert int(c100.get(3)[1]) == 99 and c100.class_names() is None
    r10 = np.zeros((2, 3073), dtype=np.uint8)
    r10[:, 0] = [4, 9]
    r10.tofile(tmp_path / "test_batch.bin")
    c10 = vision.CIFAR10.new(str(tmp_path), False)
    assert (c10.num_classes(), c10.is_train(), c10.image_size(), int(c10.get(1)[1])) == (10, False, (3, 32, 32), 9)
    cnn = vision.SimpleCNN(3, 7, 32)
    assert cnn.input_channels() == 3 and cnn.num_classes() == 7
    assert isinstance(vision.VGG.vgg13_bn(5), vision.VGG) and any("BatchNorm" in type(m).__name__ for m in vision.VGG.vgg11_bn(5).features)
    assert not any("BatchNorm" in type(m).__name__ for m in vision.VGG.vgg11(5).features)
    head = vision.VggClassifier.with_input_size(32, 3)
    assert head[0].weight.shape == (4096, 32) and head[6].weight.shape == (3, 4096)

    torch.manual_seed(0)
    tr = vision.Transformer(16, 2, 1, 1, 32, 0.0).eval()
    src, tgt = torch.randn(2, 5, 16), torch.randn(2, 4, 16)
    with torch.no_grad():
        assert tr.d_model() == 16 and tr.encoder.layers[0].d_model() == 16
        base = tr(src, tgt)
        assert torch.allclose(tr.forward_full(src, tgt), base)
        keep = torch.ones(2, 1, 1, 5, dtype=torch.bool)
        keep[..., 3:] = False                                              # the last two source positions are padding
        masked = tr.forward_full(src, tgt, src_mask=keep, memory_mask=keep)
        src2 = src.clone()
        src2[:, 3:] += 5.0
        assert torch.allclose(tr.forward_full(src2, tgt, src_mask=keep, memory_mask=keep), masked, atol=1e-5)        # masked inputs have no effect
        mem = tr.encoder.forward_with_mask(src, keep)
        mem2 = tr.encoder.forward_with_mask(src2, keep)
        assert torch.allclose(mem[:, :3], mem2[:, :3], atol=1e-5)           # visible positions ignore what is masked
        out = tr.decoder.forward_with_memory(tgt, mem, None, keep)
        out2 = tr.decoder.forward_with_memory(tgt, mem2, None, keep)
        assert torch.allclose(out, out2, atol=1e-5)
        causal = torch.ones(4, 4, dtype=torch.bool).tril()
        assert torch.allclose(tr.decoder.forward_with_memory(tgt, mem, causal, keep), out, atol=1e-5)      # the default target mask is causal
        full = torch.ones(4, 4, dtype=torch.bool)
        assert not torch.allclose(tr.decoder.forward_with_memory(tgt, mem, full, keep), out, atol=1e-5)


def test_remaining_reference_method_names():
    """Small methods the reference's types answer: one behavioural check each."""
    from axonml_b200 import autograd as ag, core, fusion, jit, parallel, profile, serialize, tensor
    from axonml_b200.core import gpu_tests as GT
    from axonml_b200.core.error import InternalError, InvalidOperation, ShapeMismatch
    assert isinstance(core.Error.shape_mismatch((2,), (3,)), ShapeMismatch) and isinstance(core.Error.invalid_operation("x"), InvalidOperation)
    assert isinstance(core.Error.internal("x"), InternalError)
    r = GT.GpuTestResult.pass_("add").with_error(1e-6).with_perf(900.0, 3.5)
    assert r.passed and r.max_abs_error == 1e-6 and (r.throughput_gbps, r.latency_us, r.error) == (900.0, 3.5, None)
    f = GT.GpuTestResult.fail("mul", "mismatch")
    rep = GT.GpuTestReport.new("cuda").with_capabilities(core.Device.Cpu().capabilities())
    rep.add_result(r); rep.add_result(f)
    assert (rep.passed_count(), rep.failed_count(), f.error, rep.backend) == (1, 1, "mismatch", "cuda") and not rep.all_passed()
    a, b = torch.randn(3, 4), torch.randn(4, 2)
    c = torch.ones(3, 2)
    core.CpuBackend.sgemm(c, a, b, 3, 2, 4, 2.0, 0.5)
    assert torch.allclose(c, 2.0 * a @ b + 0.5, atol=1e-5)
    c64 = torch.zeros(3, 2, dtype=torch.float64)
    core.CpuBackend.matmul_f64(c64, a.double(), b.double(), 3, 2, 4)
    assert torch.allclose(c64, a.double() @ b.double()) and torch.allclose(core.CpuBackend.matmul_f32(torch.empty(6), a.flatten(), b.flatten(), 3, 2, 4).view(3, 2), a @ b, atol=1e-5)
    buf = torch.empty(5)
    assert core.CpuBackend.fill(buf, 2.5).tolist() == [2.5] * 5 and core.CpuBackend.fill_zeros(buf).sum() == 0
    assert core.CpuBackend.copy(buf, torch.arange(5.0)).tolist() == [0.0, 1.0, 2.0, 3.0, 4.0]
    with pytest.raises(ValueError):
        core.CpuBackend.copy(buf, torch.zeros(4))
    assert core.CudaBackend(2).device_index() == 2

    v = ag.Variable(torch.tensor([1.0, 2.0]), True)
    assert v.ndim() == 1 and v.add(v).to_vec() == [2.0, 4.0] and v.sub(1.0).to_vec() == [0.0, 1.0] and v.mul(v).to_vec() == [1.0, 4.0] and v.div(2.0).to_vec() == [0.5, 1.0]
    assert v.sub_scalar(1.0).to_vec() == [0.0, 1.0] and v.div_scalar(4.0).to_vec() == [0.25, 0.5]
    v.set_grad([1.0, 1.0]); v.accumulate_grad(torch.tensor([0.5, 2.0]))
    assert v.grad().tolist() == [1.5, 3.0]
    v.set_grad(None)
    assert v.grad() is None
    v.accumulate_grad([1.0, 1.0])
    assert v.grad().tolist() == [1.0, 1.0]
    cl = v.clone_var()
    assert cl.requires_grad() and cl.is_leaf() and cl.tensor.data_ptr() != v.tensor.data_ptr()
    assert not ag.Variable(torch.zeros(1)).requires_grad() and ag.Variable(torch.zeros(1)).requires_grad_().requires_grad()
    assert ag.Variable.from_tensor_with_grad(torch.zeros(2)).requires_grad()
    p = ag.Variable(torch.tensor([0.8, 0.3]), True)
    p.binary_cross_entropy(torch.tensor([1.0, 0.0])).backward()
    assert p.grad() is not None
    g = ag.ComputationGraph()
    g.register_leaf(True); g.register_leaf(True)
    g.reset_id_counter()
    assert g.register_leaf(False).id == 0

    s = tensor.SparseCOO.from_coo_2d([0, 2], [1, 0], [5.0, 6.0], (3, 2)).to_csr()
    assert (s.nrows(), s.ncols(), s.nnz()) == (3, 2, 2) and s.density() == pytest.approx(1 / 3)
    assert serialize.OnnxOpType.Gelu.as_str() == "Gelu" and serialize.OnnxOpType.from_str("ReduceMin") is serialize.OnnxOpType.ReduceMin
    assert serialize.OnnxOpType.from_str("Einsum") is serialize.OnnxOpType.Unknown and len(serialize.OnnxOpType) == 32
    assert serialize.OnnxOpType.from_layer("LayerNorm") is serialize.OnnxOpType.LayerNormalization

    E = fusion.ElementwiseOp
    assert E.Relu.apply(-2.0) == 0.0 and E.Add.apply(1.0, 2.5) == 3.5 and E.Clamp.apply(5.0, 0.0, 1.0) == 1.0 and E.LeakyRelu.apply(-2.0, 0.1) == pytest.approx(-0.2)
    assert E.Square.apply(torch.tensor([2.0, -3.0])).tolist() == [4.0, 9.0] and E.Sigmoid.apply(0.0) == 0.5
    w = torch.randn(3, 2)
    assert torch.allclose(fusion.fuse_matmul_bias(w, torch.zeros(3)).forward(torch.ones(1, 2)), w.sum(1)[None], atol=1e-5)
    assert torch.equal(fusion.fused_add_relu(1.0).forward(torch.tensor([-2.0, 0.5])), torch.tensor([0.0, 1.5]))
    fc = fusion.FusionConfig.all_enabled()
    assert fc.aggressive and fc.fuse_conv and fc.min_chain_length == 2
    P = fusion.FusionPattern
    assert P.AddRelu.is_memory_bound() and P.ElementwiseChain.is_memory_bound() and not P.MatMulBiasRelu.is_memory_bound()
    opt = fusion.FusionOptimizer()
    opt.apply_fusions([(P.AddRelu, 0, 2), (P.MatMulBias, 2, 2)])
    assert opt.optimization_stats.fusions_applied == 2 and opt.optimization_stats.ops_eliminated == 2
    opt.reset_stats()
    assert opt.optimization_stats.fusions_applied == 0 and opt.optimization_stats.estimated_speedup == 1.0

    assert [d.size_bytes() for d in jit.DataType] == [4, 8, 4, 8, 1]
    gr = jit.Graph()
    i0 = gr.add_node(jit.Op.make("Constant", value=1.0), jit.DataType.F32, [2])
    n1 = gr.add_node(jit.Op.make("Neg", [i0]), jit.DataType.F32, [2])
    gr.register_input("x", i0); gr.register_output("y", n1)
    assert gr.input("x") == 0 and gr.output("y") == 1 and gr.input("z") is None and gr.topological_order() == [0, 1]
    gr.node_mut(1).shape = jit.Shape([2])
    assert gr.inputs == {"x": 0} and isinstance(gr.input("x"), jit.NodeId)

    pr = profile.Profiler()
    pr.set_enabled(False)
    pr.start("x"); pr.stop("x")
    assert not pr.is_enabled() and pr.compute.get_stats("x") is None
    pr.set_enabled(True)
    pr.compute.record("step", 4e6); pr.compute.record("step", 2e6)
    pr.record_alloc("buf", 64)
    assert pr.peak_memory() == 64 and pr.current_memory() == 64 and pr.total_time("step") == pytest.approx(6e-3) and pr.avg_time("step") == pytest.approx(3e-3)
    assert "step" in str(pr.summary()) and any(b.kind is profile.BottleneckType.SlowOperation for b in pr.analyze_bottlenecks())
    st = parallel.fsdp.FSDPMemoryStats(100, 400, 25, 200, 200, 4.0, 4)
    assert st.memory_savings() == 0.75 and st.total_memory_mb() == pytest.approx(400 / 2 ** 20) and parallel.fsdp.FSDPMemoryStats(1, 4, 1, 8, 8, 1.0).memory_savings() == 0.0
    PM = parallel.pipeline.PipelineMemoryStats
    assert PM.gpipe_peak_activations(4, 8) == 32 and PM.one_f_one_b_peak_activations(4, 8) == 4 and PM.one_f_one_b_peak_activations(4, 2) == 2
    stage = parallel.pipeline.PipelineStage(torch.nn.Linear(2, 3), 1, 0)
    assert stage.forward(torch.zeros(1, 2)).shape == (1, 3) and stage(torch.zeros(1, 2)).shape == (1, 3)
    gb = parallel.GradientBucket(8)
    assert gb.data_mut().numel() == 0


def test_tensor_module_functions_named_after_the_reference_methods():
    import axonml_b200.tensor as T
    from axonml_b200.core import Storage
    x = T.from_slice(range(12), [3, 4])
    assert T.slice(x, [(1, 3), (0, 2)]).tolist() == [[4, 5], [8, 9]]
    assert T.get(x, [2, 3]) == 11 and T.to_vec(T.slice_dim0(x, 0, 1)) == [0, 1, 2, 3]
    with pytest.raises(IndexError):
        T.get(x, [1])
    assert T.strides(x.t()) == [1, 4] and T.clone_deep(x.t()).is_contiguous()
    assert T.is_scalar(T.scalar(1.0)) and T.is_empty(T.zeros([0])) and not T.is_empty(x)
    assert T.mean_dim(x, 1).tolist() == [1.5, 5.5, 9.5]
    assert T.from_storage(Storage(torch.arange(6.0)), [2, 3]).tolist() == [[0, 1, 2], [3, 4, 5]]
    assert T.to_device(x, "cpu").shape == (3, 4)
