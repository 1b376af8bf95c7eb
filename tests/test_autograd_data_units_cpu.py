"""Unit tests of the autograd facade and the data pipeline on the CPU, one behaviour per test (the
topics of the reference's in-module tests under crates/axonml-autograd/src and
crates/axonml-data/src)."""
import threading

import pytest
import torch

from axonml_b200 import autograd as A, data as D
from axonml_b200.autograd import Variable


# -------------------------------------------------------------------------------------- variables
def test_variable_creation_and_leaf_flags():
    v = Variable.new(torch.tensor([1.0, 2.0]), True)
    assert v.requires_grad() and v.is_leaf() and v.shape() == (2,) and v.numel() == 2 and v.grad() is None
    w = Variable.from_tensor(torch.zeros(3))
    assert not w.requires_grad() and w.to_vec() == [0.0] * 3


def test_variable_arithmetic_builds_a_graph():
    a, b = Variable(torch.tensor([1.0, 2.0]), True), Variable(torch.tensor([3.0, 4.0]), True)
    c = a.add_var(b).mul_var(a).sum()
    assert not c.is_leaf() and c.grad_fn() is not None and c.item() == 4.0 + 12.0
    c.backward()
    assert a.grad().tolist() == [5.0, 8.0] and b.grad().tolist() == [1.0, 2.0]


def test_variable_detach_cuts_the_graph():
    a = Variable(torch.tensor([2.0]), True)
    d = a.mul_scalar(3.0).detach()
    assert not d.requires_grad() and d.grad_fn() is None and d.item() == 6.0


def test_variable_gradients_accumulate_until_zeroed():
    a = Variable(torch.tensor([1.0, 1.0]), True)
    a.mul_scalar(2.0).sum().backward()
    a.mul_scalar(3.0).sum().backward()
    assert a.grad().tolist() == [5.0, 5.0]
    a.zero_grad()
    assert a.grad() is None
    a.set_grad(torch.ones(2))
    a.accumulate_grad(torch.ones(2))
    assert a.grad().tolist() == [2.0, 2.0]


def test_chain_rule_through_several_operations():
    x = Variable(torch.tensor([0.5, -0.3]), True)
    y = x.mul_scalar(2.0).tanh().pow(2).sum()
    y.backward()
    t = torch.tanh(torch.tensor([1.0, -0.6]))
    assert torch.allclose(x.grad(), 2 * t * (1 - t ** 2) * 2, atol=1e-6)


def test_variable_mse_loss():
    p, t = Variable(torch.tensor([1.0, 2.0, 3.0]), True), torch.tensor([1.0, 1.0, 1.0])
    loss = p.mse_loss(t)
    assert loss.item() == pytest.approx(5 / 3)
    loss.backward()
    assert torch.allclose(p.grad(), torch.tensor([0.0, 2 / 3, 4 / 3]))


@pytest.mark.parametrize("fn", [
    lambda x: (x * x).sum(), lambda x: x.pow(3).mean(), lambda x: torch.sigmoid(x).sum(), lambda x: torch.tanh(x).sum(),
    lambda x: torch.nn.functional.leaky_relu(x, 0.1).sum(), lambda x: (x.reshape(2, 3) @ x.reshape(3, 2)).sum(),
    lambda x: x.reshape(2, 3).t().exp().sum(), lambda x: (x - 1.0).abs().sum()])
def test_gradcheck_passes_on_smooth_functions(fn):
    x = torch.tensor([0.3, -0.7, 1.1, 0.9, -1.3, 0.2])
    assert A.gradcheck(fn, x)


def test_numerical_gradient_of_a_quadratic():
    g = A.numerical_gradient(lambda x: (x ** 2).sum(), torch.tensor([1.0, -2.0, 3.0]))
    assert torch.allclose(g.float(), torch.tensor([2.0, -4.0, 6.0]), atol=1e-4)


def test_gradcheck_fails_on_a_wrong_gradient():
    class Wrong(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x): return x * 2
        @staticmethod
        def backward(ctx, g): return g * 3
    assert not A.gradcheck(lambda x: Wrong.apply(x).sum(), torch.tensor([1.0, 2.0]))


# -------------------------------------------------------------------------------------- grad mode
def test_grad_is_enabled_by_default_and_no_grad_nests():
    assert A.is_grad_enabled()
    with A.no_grad():
        assert not A.is_grad_enabled()
        with A.no_grad():
            assert not A.is_grad_enabled()
        assert not A.is_grad_enabled()
        with A.enable_grad():
            assert A.is_grad_enabled()
        assert not A.is_grad_enabled()
    assert A.is_grad_enabled()


def test_no_grad_results_carry_no_graph():
    x = torch.ones(2, requires_grad=True)
    with A.no_grad():
        y = x * 2
    assert not y.requires_grad
    with A.inference_mode():
        assert A.is_inference_mode() and not A.is_grad_enabled()
    assert not A.is_inference_mode()


def test_guard_objects_restore_the_previous_mode():
    g = A.NoGradGuard()
    assert not A.is_grad_enabled()
    e = A.EnableGradGuard()
    assert A.is_grad_enabled()
    e.drop()
    assert not A.is_grad_enabled()
    g.drop()
    assert A.is_grad_enabled()


# --------------------------------------------------------------------------------------- autocast
def test_autocast_is_off_by_default_and_guards_nest():
    assert not A.is_autocast_enabled() and A.autocast_depth() == 0
    with A.autocast(torch.bfloat16):
        assert A.is_autocast_enabled() and A.autocast_depth() == 1 and str(A.autocast_dtype()) == "bf16"
        with A.autocast(torch.float16):
            assert A.autocast_depth() == 2 and str(A.autocast_dtype()) == "f16"
        assert str(A.autocast_dtype()) == "bf16"
        with A.disable_autocast():
            assert not A.is_autocast_enabled()
        assert A.is_autocast_enabled()
    assert not A.is_autocast_enabled() and A.autocast_depth() == 0


def test_autocast_lowers_matmul_and_keeps_reductions():
    a, b = torch.randn(4, 4), torch.randn(4, 4)
    with A.autocast(torch.bfloat16):
        assert (a @ b).dtype == torch.bfloat16 and torch.softmax(a, -1).dtype == torch.float32
    assert (a @ b).dtype == torch.float32
    assert {p.name for p in A.AutocastPolicy} == {"LowerPrecision", "FullPrecision", "Promote"}


def test_autocast_depth_is_per_thread():
    seen = []
    with A.autocast(torch.bfloat16):
        t = threading.Thread(target=lambda: seen.append(A.autocast_depth()))
        t.start()
        t.join()
        assert A.autocast_depth() == 1
    assert seen == [0]


# ------------------------------------------------------------------------------------ checkpointing
def test_checkpoint_gives_the_same_values_and_gradients():
    lin = torch.nn.Linear(4, 4)
    f = lambda x: torch.tanh(lin(x)).pow(2)
    x1, x2 = torch.randn(3, 4, requires_grad=True), None
    x2 = x1.detach().clone().requires_grad_(True)
    f(x1).sum().backward()
    g_ref = lin.weight.grad.clone()
    lin.zero_grad()
    A.checkpoint(f, x2).sum().backward()
    assert torch.allclose(x1.grad, x2.grad) and torch.allclose(lin.weight.grad, g_ref)


def test_checkpoint_recomputes_the_forward_during_backward():
    calls = []
    def f(x):
        calls.append(1)
        return x.sin()
    x = torch.randn(5, requires_grad=True)
    y = A.checkpoint(f, x)
    assert len(calls) == 1
    y.sum().backward()
    assert len(calls) == 2
    with A.no_grad():
        A.checkpoint(f, x)
    assert len(calls) == 3


@pytest.mark.parametrize("segments", [0, 1, 2, 3, 6, 9])
def test_checkpoint_sequential_matches_the_plain_stack(segments):
    torch.manual_seed(0)
    layers = [torch.nn.Linear(4, 4) for _ in range(6)]
    run = lambda i, x: torch.relu(layers[i](x))
    x = torch.randn(2, 4, requires_grad=True)
    ref = x
    for i in range(6):
        ref = run(i, ref)
    out = A.checkpoint_sequential(6, segments, x, run)
    assert torch.allclose(out, ref, atol=1e-6)
    out.sum().backward()
    assert x.grad is not None


def test_memory_estimates_and_segment_suggestions():
    assert A.estimate_memory_savings(12, 4, 10.0) == (120.0, 30.0)
    assert A.estimate_memory_savings(12, 0, 10.0) == (120.0, 120.0)
    assert A.suggest_segments(10, 1.0, 100.0) == 0          # everything fits
    assert A.suggest_segments(12, 10.0, 40.0) == 3          # four activations fit -> three segments
    assert A.suggest_segments(8, 10.0, 5.0) == 8            # not even one fits


# ------------------------------------------------------------------------------------------ graph
def test_graph_nodes_leaf_and_intermediate():
    x = torch.ones(2, requires_grad=True)
    y = (x * 2).sum()
    g = A.ComputationGraph.from_output(y)
    dot = g.to_dot()
    assert "digraph" in dot and "Sum" in dot and "Mul" in dot
    leaf = A.GraphNode.leaf(True, 7)
    assert leaf.is_leaf and leaf.grad_fn is None and leaf.topo_order == 0 and leaf.id == 7
    inner = A.GraphNode.intermediate(A.GradFn.of(y) if hasattr(A.GradFn, "of") else None, True, 2)
    assert not inner.is_leaf and inner.topo_order == 2


def test_named_backward_functions_follow_the_formulas():
    g = torch.tensor([1.0, 2.0])
    a, b = torch.tensor([3.0, 4.0]), torch.tensor([5.0, 6.0])
    add = A.AddBackward()
    assert add.forward(a, b).tolist() == [8.0, 10.0] and [t.tolist() for t in add.apply(g)] == [[1.0, 2.0], [1.0, 2.0]]
    mul = A.MulBackward()
    mul.forward(a, b)
    ga, gb = mul.apply(g)
    assert ga.tolist() == [5.0, 12.0] and gb.tolist() == [3.0, 8.0]
    relu = A.ReluBackward()
    relu.forward(torch.tensor([-1.0, 1.0]))
    gr = relu.apply(g)
    assert (gr[0] if isinstance(gr, tuple) else gr).tolist() == [0.0, 2.0]
    x = torch.tensor([0.5, -0.5], requires_grad=True)
    A.TanhBackward.call(x).sum().backward()                 # through the tape
    assert torch.allclose(x.grad, 1 - torch.tanh(x.detach()) ** 2)
    assert A.sum_to_shape(torch.ones(2, 3), (3,)).tolist() == [2.0, 2.0, 2.0]
    assert A.sum_to_shape(torch.ones(2, 3), (2, 1)).tolist() == [[3.0], [3.0]]


# --------------------------------------------------------------------------------------- datasets
def _ds(n=10):
    return D.TensorDataset(torch.arange(n * 2.0).reshape(n, 2), torch.arange(n))


def test_tensor_dataset_indexing():
    ds = _ds()
    assert ds.len() == 10 and not ds.is_empty()
    x, y = ds.get(3)
    assert x.tolist() == [6.0, 7.0] and int(y) == 3
    with pytest.raises((IndexError, Exception)):
        ds.get(10)


def test_map_concat_subset_in_memory_datasets():
    ds = _ds(4)
    m = D.MapDataset(ds, lambda x, y: (x * 2, y))
    assert m.get(1)[0].tolist() == [4.0, 6.0] and m.len() == 4
    c = D.ConcatDataset([ds, _ds(3)])
    assert c.len() == 7 and int(c.get(5)[1]) == 1
    s = D.SubsetDataset(ds, [3, 1])
    assert s.len() == 2 and int(s.get(0)[1]) == 3
    mem = D.InMemoryDataset([(torch.zeros(1), torch.tensor(0))])
    mem.push((torch.ones(1), torch.tensor(1)))
    assert mem.len() == 2 and int(mem.get(1)[1]) == 1


def test_random_split_partitions_the_dataset():
    parts = D.random_split(_ds(10), [7, 3])
    assert [p.len() for p in parts] == [7, 3]
    seen = sorted(int(p.get(i)[1]) for p in parts for i in range(p.len()))
    assert seen == list(range(10))


# --------------------------------------------------------------------------------------- samplers
def test_sequential_and_random_samplers():
    assert list(D.SequentialSampler(5)) == [0, 1, 2, 3, 4]
    r = list(D.RandomSampler(50))
    assert sorted(r) == list(range(50)) and r != list(range(50))
    w = list(D.RandomSampler.with_replacement(5, 40))
    assert len(w) == 40 and set(w) <= set(range(5))


def test_subset_and_weighted_samplers():
    s = list(D.SubsetRandomSampler([2, 4, 6]))
    assert sorted(s) == [2, 4, 6]
    w = list(D.WeightedRandomSampler([0.0, 1.0, 0.0], 20))
    assert w == [1] * 20
    torch.manual_seed(0)
    heavy = list(D.WeightedRandomSampler([0.9, 0.1], 500))
    assert heavy.count(0) > 350


def test_batch_sampler_with_and_without_drop_last():
    b = D.BatchSampler(D.SequentialSampler(7), 3)
    assert list(b) == [[0, 1, 2], [3, 4, 5], [6]] and b.len() == 3
    d = D.BatchSampler(D.SequentialSampler(7), 3, drop_last=True)
    assert list(d) == [[0, 1, 2], [3, 4, 5]] and d.len() == 2 and not d.is_empty()


def test_distributed_sampler_shards_are_disjoint_and_cover():
    shards = [list(D.DistributedSampler(10, 2, r, shuffle=False)) for r in range(2)]
    assert len(shards[0]) == len(shards[1]) == 5 and sorted(shards[0] + shards[1]) == list(range(10))
    a = D.DistributedSampler(10, 2, 0, shuffle=True, seed=1)
    a.set_epoch(0)
    e0 = list(a)
    a.set_epoch(1)
    assert list(a) != e0


# ---------------------------------------------------------------------------------------- loaders
def test_dataloader_batches_in_order():
    dl = D.DataLoader(_ds(10), batch_size=4)
    batches = list(dl)
    assert dl.len() == 3 and [b.size for b in batches] == [4, 4, 2] and dl.dataset_len() == 10
    assert torch.cat([b.targets for b in batches]).tolist() == list(range(10))
    assert batches[0].data.shape == (4, 2) and batches[0].len() == 4 and not batches[0].is_empty()


def test_dataloader_drop_last_and_exact_batches():
    assert [b.size for b in D.DataLoader(_ds(10), 4, drop_last=True)] == [4, 4]
    assert D.DataLoader(_ds(10), 4, drop_last=True).len() == 2
    assert [b.size for b in D.DataLoader(_ds(8), 4)] == [4, 4]


def test_dataloader_shuffle_permutes_but_keeps_every_sample():
    torch.manual_seed(0)
    dl = D.DataLoader(_ds(64), 8, shuffle=True)
    order = torch.cat([b.targets for b in dl]).tolist()
    assert sorted(order) == list(range(64)) and order != list(range(64))
    assert order != torch.cat([b.targets for b in dl]).tolist()          # a new order each pass


def test_dataloader_empty_and_single_item():
    empty = D.DataLoader(D.TensorDataset(torch.zeros(0, 2), torch.zeros(0)), 4)
    assert list(empty) == [] and empty.is_empty() and empty.len() == 0
    one = list(D.DataLoader(_ds(1), 4))
    assert len(one) == 1 and one[0].size == 1


def test_dataloader_iterator_counts_what_is_left():
    it = D.DataLoader(_ds(10), 4).iter()
    assert it.remaining() == 3
    next(it)
    assert it.remaining() == 2 and len(list(it)) == 2 and it.remaining() == 0


def test_worker_threads_give_the_same_batches_as_the_sequential_loader():
    seq = [b.data for b in D.DataLoader(_ds(37), 5)]
    par = [b.data for b in D.DataLoader(_ds(37), 5, num_workers=3)]
    assert len(seq) == len(par) and all(a.equal(b) for a, b in zip(seq, par))
    assert [b.size for b in D.DataLoader(_ds(37), 5, num_workers=2, drop_last=True)] == [5] * 7


def test_generic_dataloader_uses_the_collate_function():
    samples = D.InMemoryDataset([torch.full((2,), float(i)) for i in range(5)])
    out = list(D.GenericDataLoader(samples, 2, collate=D.StackCollate()))
    assert [tuple(o.shape) for o in out] == [(2, 2), (2, 2), (1, 2)] and out[1][0].tolist() == [2.0, 2.0]


# ---------------------------------------------------------------------------------------- collate
def test_stack_and_concat_helpers():
    a, b = torch.ones(2), torch.zeros(2)
    assert D.stack_tensors([a, b]).shape == (2, 2) and D.stack_tensors([torch.ones(2, 3)] * 4).shape == (4, 2, 3)
    assert D.concat_tensors([a, b]).tolist() == [1, 1, 0, 0] and D.concat_tensors([torch.ones(1, 2), torch.ones(1, 3)], 1).shape == (1, 5)


def test_default_and_stack_collate():
    pairs = [(torch.full((3,), float(i)), torch.tensor(i)) for i in range(4)]
    x, y = D.DefaultCollate().collate(pairs)
    assert x.shape == (4, 3) and y.tolist() == [0, 1, 2, 3]
    assert D.StackCollate.with_dim(1).collate([torch.ones(2), torch.zeros(2)]).tolist() == [[1, 0], [1, 0]]


# ------------------------------------------------------------------------------------- transforms
def test_normalize_scale_clamp():
    x = torch.tensor([0.0, 0.5, 1.0])
    assert D.Normalize(0.5, 0.5).apply(x).tolist() == [-1.0, 0.0, 1.0] and D.Normalize.zero_centered().apply(x).tolist() == [-1.0, 0.0, 1.0]
    assert D.Normalize.standard().apply(x).equal(x)
    img = torch.ones(2, 2, 2)
    assert D.Normalize([1.0, 0.0], [1.0, 2.0]).apply(img)[:, 0, 0].tolist() == [0.0, 0.5]
    assert D.Scale(2.0).apply(x).tolist() == [0.0, 1.0, 2.0]
    y = torch.tensor([-2.0, 0.3, 2.0])
    assert D.Clamp(-1.0, 1.0).apply(y).tolist() == pytest.approx([-1.0, 0.3, 1.0])
    assert D.Clamp.zero_one().apply(y).tolist() == pytest.approx([0.0, 0.3, 1.0]) and D.Clamp.symmetric().apply(y).tolist() == pytest.approx([-1.0, 0.3, 1.0])


def test_flatten_reshape_lambda_to_tensor():
    x = torch.arange(6.0).reshape(2, 3)
    assert D.Flatten().apply(x).shape == (6,) and D.Reshape([3, 2]).apply(x).shape == (3, 2)
    assert D.Lambda(lambda t: t + 1).apply(x)[0, 0].item() == 1.0
    assert D.ToTensor().apply([1, 2, 3]).dtype == torch.float32


def test_compose_applies_in_order_and_builds_incrementally():
    c = D.Compose([D.Scale(2.0), D.Lambda(lambda t: t + 1)])
    assert c.apply(torch.tensor([1.0])).item() == 3.0 and c.len() == 2
    e = D.Compose.empty()
    assert e.is_empty() and e.apply(torch.tensor([5.0])).item() == 5.0
    e.add(D.Scale(3.0))
    assert e.apply(torch.tensor([5.0])).item() == 15.0


def test_random_transforms_keep_shape_and_statistics():
    torch.manual_seed(0)
    x = torch.zeros(10000)
    n = D.RandomNoise(0.1).apply(x)
    assert n.shape == x.shape and abs(float(n.std()) - 0.1) < 0.01
    d = D.DropoutTransform(0.3).apply(torch.ones(10000))
    assert 0.25 < float((d == 0).float().mean()) < 0.35
    v = torch.arange(4.0)
    assert D.RandomFlip(-1, 1.0).apply(v).tolist() == [3, 2, 1, 0] and D.RandomFlip(-1, 0.0).apply(v).equal(v)
    img = torch.arange(6.0).reshape(1, 2, 3)
    assert D.RandomFlip(-2, 1.0).apply(img).tolist() == [[[3, 4, 5], [0, 1, 2]]]


def test_random_crop_sizes():
    img = torch.randn(3, 10, 12)
    assert D.RandomCrop(8).apply(img).shape == (3, 8, 8) and D.RandomCrop.new_2d(4, 6).apply(img).shape == (3, 4, 6)
    assert D.RandomCrop(20).apply(img).shape == (3, 10, 12)          # larger than the image: unchanged
    assert D.RandomCrop((1, 5)).apply(torch.arange(9.0).reshape(1, 9)).shape == (1, 5)
