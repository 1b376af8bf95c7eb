"""Unit tests of the distributed layer on the in-process mock backend (one rank, and worlds of threads),
one behaviour per test (the topics of the reference's in-module and integration tests under
crates/axonml-distributed).  The multi-process paths over gloo live in test_distributed_cpu.py."""
import threading

import pytest
import torch

from axonml_b200 import nn, parallel as PL
from axonml_b200.parallel import MockBackend, ProcessGroup, ReduceOp, World


def _world(n, fn, timeout_s=5.0):
    """Runs ``fn(rank, ProcessGroup)`` on ``n`` threads sharing one mock world; returns the results by rank."""
    backends = MockBackend.create_world(n, timeout_s=timeout_s)
    out, errs = [None] * n, []

    def go(r):
        try:
            out[r] = fn(r, ProcessGroup(backends[r]))
        except Exception as e:  # noqa: BLE001 - reported to the test below
            errs.append(e)
    threads = [threading.Thread(target=go, args=(r,)) for r in range(n)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    if errs:
        raise errs[0]
    return out


# ------------------------------------------------------------------------------------ groups
def test_mock_backend_single_rank():
    be = MockBackend.single()
    assert be.rank() == 0 and be.world_size() == 1 and be.name() == "mock"
    t = torch.tensor([1.0, 2.0])
    be.all_reduce(t, ReduceOp.Sum)
    assert t.tolist() == [1.0, 2.0]
    be.barrier()


def test_process_group_mock_and_membership():
    pg = ProcessGroup.mock()
    assert pg.rank() == 0 and pg.world_size() == 1 and pg.size() == 1 and pg.ranks() == [0]
    assert pg.contains(0) and not pg.contains(1)
    assert PL.rank(pg) == 0 and PL.world_size(pg) == 1 and PL.is_main_process(pg)
    pg.barrier()
    PL.barrier(pg)


def test_world_default_group_and_subgroups():
    w = World.mock()
    assert w.rank() == 0 and w.world_size() == 1 and w.is_main() and w.default_group().size() == 1
    sub = w.new_group([0])
    assert sub is not None and sub.contains(0)
    w.barrier()


def test_reduce_op_variants():
    assert {o.name for o in ReduceOp} == {"Sum", "Product", "Min", "Max", "Average"}


@pytest.mark.parametrize("op,expect", [(ReduceOp.Sum, [6.0, 9.0]), (ReduceOp.Product, [6.0, 24.0]), (ReduceOp.Min, [1.0, 2.0]),
                                       (ReduceOp.Max, [3.0, 4.0]), (ReduceOp.Average, [2.0, 3.0])])
def test_all_reduce_every_operation_over_three_ranks(op, expect):
    data = [[1.0, 2.0], [2.0, 3.0], [3.0, 4.0]]

    def fn(r, pg):
        t = torch.tensor(data[r])
        pg.backend().all_reduce(t, op)
        return t.tolist()
    assert _world(3, fn) == [expect] * 3


def test_functional_all_reduce_helpers():
    def fn(r, pg):
        t = torch.tensor([float(r + 1)])
        return [PL.all_reduce_sum(t.clone(), pg).item(), PL.all_reduce_mean(t.clone(), pg).item(),
                PL.all_reduce_min(t.clone(), pg).item(), PL.all_reduce_max(t.clone(), pg).item(),
                PL.all_reduce_product(t.clone(), pg).item()]
    assert _world(2, fn) == [[3.0, 1.5, 1.0, 2.0, 2.0]] * 2


def test_broadcast_from_any_root():
    def fn(r, pg):
        a = PL.broadcast(torch.tensor([float(r)]), pg)
        b = PL.broadcast_from(torch.tensor([float(r * 10)]), 2, pg)
        return a.item(), b.item()
    assert _world(3, fn) == [(0.0, 20.0)] * 3


def test_all_gather_and_reduce_scatter():
    def fn(r, pg):
        g = PL.all_gather(torch.tensor([float(r), float(r)]), pg)
        rs = PL.reduce_scatter_sum(torch.arange(4.0) + r, pg)
        rm = PL.reduce_scatter_mean(torch.arange(4.0) + r, pg)
        return g.flatten().tolist(), rs.tolist(), rm.tolist()
    out = _world(2, fn)
    assert out[0][0] == out[1][0] == [0.0, 0.0, 1.0, 1.0]
    assert out[0][1] == [1.0, 3.0] and out[1][1] == [5.0, 7.0] and out[0][2] == [0.5, 1.5]


def test_scatter_and_gather_tensor_round_trip():
    def fn(r, pg):
        full = torch.arange(8.0).reshape(4, 2)
        mine = PL.scatter_tensor(full, pg)
        back = PL.gather_tensor(mine, pg)
        return mine.tolist(), back.equal(full)
    out = _world(2, fn)
    assert out[0] == ([[0.0, 1.0], [2.0, 3.0]], True) and out[1] == ([[4.0, 5.0], [6.0, 7.0]], True)


def test_send_recv_between_two_ranks():
    def fn(r, pg):
        if r == 0:
            pg.send_tensor(torch.tensor([7.0, 8.0]), 1)
            return None
        return pg.recv_tensor(0, (2,)).tolist()
    assert _world(2, fn)[1] == [7.0, 8.0]


def test_ring_all_reduce_equals_the_direct_sum():
    def fn(r, pg):
        t = torch.arange(10.0) * (r + 1)
        return PL.ring_all_reduce(t.clone(), pg).tolist(), PL.ring_all_reduce(t.clone(), pg, ReduceOp.Average).tolist()
    out = _world(4, fn)
    assert all(o[0] == (torch.arange(10.0) * 10).tolist() for o in out)
    assert all(o[1] == (torch.arange(10.0) * 2.5).tolist() for o in out)


def test_sync_gradients_averages_across_ranks():
    def fn(r, pg):
        one = PL.sync_gradient(torch.full((3,), float(r)), pg)
        many = PL.sync_gradients([torch.full((2,), float(r)), torch.full((1,), 2.0 * r)], pg)
        return one.tolist(), [m.tolist() for m in many]
    out = _world(2, fn)
    assert out[0] == out[1] == ([0.5] * 3, [[0.5, 0.5], [1.0]])


def test_a_dropped_message_times_out_instead_of_hanging():
    backends = MockBackend.create_world(2, timeout_s=0.3)
    backends[0].drop_next_message(0, 1)
    backends[0].send(torch.ones(2), 1)
    with pytest.raises(PL.CommTimeout):
        backends[1].recv(torch.empty(2), 0)


def test_subgroups_reduce_only_among_their_members():
    def fn(r, pg):
        g = pg.backend().new_group([0, 1] if r < 2 else [2, 3])
        t = torch.tensor([float(r)])
        g.all_reduce(t, ReduceOp.Sum)
        return t.item()
    assert _world(4, fn) == [1.0, 1.0, 5.0, 5.0]


# ----------------------------------------------------------------------------- gradient buckets
def test_gradient_bucket_add_extract_clear():
    b = PL.GradientBucket.new(10)
    assert b.is_empty() and b.capacity() == 10 and not b.is_full()
    assert b.add(torch.ones(2, 3)) and b.add(torch.full((4,), 2.0))
    assert b.size() == 10 and b.is_full() and b.num_tensors() == 2 and not b.add(torch.ones(1))
    assert b.data().tolist() == [1.0] * 6 + [2.0] * 4
    b.data_mut().mul_(2.0)
    a, c = b.extract()
    assert a.shape == (2, 3) and a.unique().tolist() == [2.0] and c.tolist() == [4.0] * 4
    b.clear()
    assert b.is_empty() and b.num_tensors() == 0


def test_gradient_synchronizer_averages_in_buckets():
    def fn(r, pg):
        s = PL.GradientSynchronizer.new(PL.GradSyncStrategy.Synchronous, 4)
        grads = [torch.full((3,), float(r)), torch.full((2, 2), 2.0 * r), torch.full((1,), 4.0 * r)]
        s.prepare(len(grads))
        for i, g in enumerate(grads):
            s.add_gradient(i, g)
        s.sync_all(pg)
        return [g.flatten().tolist() for g in grads]
    out = _world(2, fn)
    assert out[0] == out[1] == [[0.5] * 3, [1.0] * 4, [2.0]]


def test_gradient_synchronizer_no_sync_leaves_gradients_alone():
    s = PL.GradientSynchronizer(PL.GradSyncStrategy.NoSync)
    g = torch.ones(3)
    s.prepare(1)
    s.add_gradient(0, g)
    s.sync_all(ProcessGroup.mock())
    assert g.tolist() == [1.0] * 3 and s.strategy() is PL.GradSyncStrategy.NoSync
    assert PL.GradientSynchronizer().strategy() is PL.GradSyncStrategy.Synchronous


# ------------------------------------------------------------------------------------------ DDP
def _mlp():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 2))


def test_ddp_wraps_forwards_and_exposes_the_module():
    m = _mlp()
    ddp = PL.DDP(m, ProcessGroup.mock())
    x = torch.randn(3, 4)
    assert torch.allclose(ddp(x), m(x)) and ddp.module() is m
    assert len(list(ddp.parameters())) == 4
    ddp.eval()
    assert not m.training
    ddp.train()
    assert m.training


def test_ddp_gradients_are_averaged_over_ranks():
    state = _mlp().state_dict()                      # built once: the global generator is not per thread

    def model():
        m = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 2))
        m.load_state_dict(state)
        return m

    def fn(r, pg):
        ddp = PL.DDP(model(), pg, fused=False)
        ddp.sync_parameters()
        ddp(torch.full((2, 4), float(r + 1))).sum().backward()
        return [p.grad.clone() for p in ddp.parameters()]
    out = _world(2, fn)
    ref = []
    for r in range(2):
        m = model()
        m(torch.full((2, 4), float(r + 1))).sum().backward()
        ref.append([p.grad for p in m.parameters()])
    for g0, g1, a, b in zip(out[0], out[1], ref[0], ref[1]):
        assert torch.allclose(g0, g1) and torch.allclose(g0, (a + b) / 2, atol=1e-6)


def test_ddp_no_sync_keeps_local_gradients():
    state = _mlp().state_dict()

    def fn(r, pg):
        m = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 2))
        m.load_state_dict(state)
        ddp = PL.DDP(m, pg, fused=False)
        with ddp.no_sync():
            ddp(torch.full((2, 4), float(r + 1))).sum().backward()
        return m[0].weight.grad.clone()
    a, b = _world(2, fn)
    assert not torch.allclose(a, b)


# ----------------------------------------------------------------------------------------- FSDP
def test_sharding_strategies_and_offload_modes():
    assert {s.name for s in PL.ShardingStrategy} == {"FullShard", "ShardGradOp", "NoShard", "HybridShard"}
    assert {c.name for c in PL.CPUOffload} == {"None_", "Params", "Full"}


def test_fsdp_memory_statistics():
    st = PL.FSDPMemoryStats(total_params=1000, total_param_memory=4000, local_params=250, local_param_memory=1000,
                            local_optimizer_memory=2000, savings_factor=4.0, world_size=4)
    assert st.memory_savings() == pytest.approx(0.75) and st.total_memory_mb() == pytest.approx(3000 / 1024 / 1024)
    assert PL.FSDPMemoryStats(10, 40, 10, 40, 80, 1.0).memory_savings() == 0.0


def test_fsdp_single_rank_matches_the_plain_module():
    m = _mlp()
    ref = _mlp()
    f = PL.FSDP(m, ProcessGroup.mock(), device="cpu")
    x = torch.randn(5, 4)
    assert torch.allclose(f(x), ref(x), atol=1e-6)
    est = f.memory_estimate()
    assert est.total_params == sum(p.numel() for p in ref.parameters()) and est.world_size == 1


# ------------------------------------------------------------------------------ tensor parallel
def test_column_and_row_parallel_linear_on_one_rank_equal_a_linear():
    pg = ProcessGroup.mock()
    col, row = PL.ColumnParallelLinear(6, 8, process_group=pg, gather_output=True), PL.RowParallelLinear(8, 3, process_group=pg, input_is_parallel=True)
    x = torch.randn(4, 6)
    h = col(x)
    assert h.shape == (4, 8) and torch.allclose(h, torch.nn.functional.linear(x, col.weight, col.bias), atol=1e-5)
    assert torch.allclose(row(h), torch.nn.functional.linear(h, row.weight, row.bias), atol=1e-5)


def test_column_then_row_parallel_over_two_ranks_equals_the_dense_pair():
    torch.manual_seed(1)
    W1, b1, W2, b2, x = torch.randn(8, 6), torch.randn(8), torch.randn(3, 8), torch.randn(3), torch.randn(4, 6)

    def fn(r, pg):
        col, row = PL.ColumnParallelLinear(6, 8, process_group=pg), PL.RowParallelLinear(8, 3, process_group=pg)
        with torch.no_grad():
            col.weight.copy_(W1[r * 4:(r + 1) * 4]), col.bias.copy_(b1[r * 4:(r + 1) * 4])
            row.weight.copy_(W2[:, r * 4:(r + 1) * 4]), row.bias.copy_(b2)
        return row(torch.relu(col(x)))
    out = _world(2, fn)
    ref = torch.relu(x @ W1.t() + b1) @ W2.t() + b2
    assert torch.allclose(out[0], ref, atol=1e-5) and torch.allclose(out[1], ref, atol=1e-5)


# ------------------------------------------------------------------------------------ pipeline
def test_pipeline_schedules_and_memory_statistics():
    assert {s.name for s in PL.PipelineSchedule} == {"GPipe", "OneFOneBSchedule", "InterleavedOneFOneB"}
    S = PL.PipelineMemoryStats
    assert S.gpipe_peak_activations(4, 8) == 32 and S.one_f_one_b_peak_activations(4, 8) == 4 and S.one_f_one_b_peak_activations(4, 2) == 2


def test_pipeline_stage_and_microbatch_split():
    stage = PL.PipelineStage(nn.Linear(4, 4), 0, 0)
    assert stage.stage_id == 0 and stage.device_rank == 0 and stage(torch.randn(2, 4)).shape == (2, 4)
    pipe = PL.Pipeline([stage], ProcessGroup.mock(), PL.PipelineSchedule.GPipe, num_microbatches=4)
    parts = pipe.split_microbatches(torch.arange(16.0).reshape(8, 2))
    assert len(parts) == 4 and all(p.shape == (2, 2) for p in parts)
    assert pipe.combine_microbatches(parts).equal(torch.arange(16.0).reshape(8, 2))


def test_device_mesh_coordinates_and_groups():
    def fn(r, pg):
        mesh = PL.DeviceMesh(World(pg.backend()), {"dp": 2, "tp": 2})
        return mesh.coord("dp"), mesh.coord("tp"), mesh.group("tp").ranks(), mesh.size("dp")
    out = _world(4, fn)
    assert [o[:2] for o in out] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert out[0][2] == [0, 1] and out[3][2] == [2, 3] and out[0][3] == 2
