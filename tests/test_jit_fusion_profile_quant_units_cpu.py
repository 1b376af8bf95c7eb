"""Unit tests of the graph compiler, the fusion library, the profiler and the block quantiser on the
CPU, one behaviour per test (the topics of the reference's in-module tests under crates/axonml-jit,
crates/axonml-fusion, crates/axonml-profile and crates/axonml-quant)."""
import json
import time

import pytest
import torch

from axonml_b200 import fusion as FU, jit as J, profile as P, quant as Q


# -------------------------------------------------------------------------------------- tracing
def _chain(t):
    x = t.input("x", [2, 3])
    return t.output("y", x.relu().mul_scalar(2.0).add_scalar(1.0))


def test_trace_records_inputs_operations_and_outputs():
    g = J.trace(_chain)
    assert g.input_names() == ["x"] and g.output_names() == ["y"] and g.len() == 5
    kinds = [n.op.kind for n in g.nodes]
    assert kinds[0] == "Input" and kinds[-1] == "Output" and "Relu" in kinds
    assert tuple(g.node(g.output("y")).shape.dims()) == (2, 3)


def test_trace_matmul_and_reduction_shapes():
    def f(t):
        a, b = t.input("a", [4, 5]), t.input("b", [5, 6])
        m = a.matmul(b)
        t.output("m", m)
        t.output("s", m.mean_axis(1) if hasattr(m, "mean_axis") else m.mean())
    g = J.trace(f)
    assert tuple(g.node(g.output("m")).shape.dims()) == (4, 6)
    assert tuple(g.node(g.output("s")).shape.dims()) in ((4,), (4, 1))


def test_interpreter_matches_torch_on_a_chain():
    g = J.trace(_chain)
    x = torch.randn(2, 3)
    assert torch.allclose(J.interpret(g, {"x": x})["y"], torch.relu(x) * 2 + 1)


def test_compiled_model_runs_and_reports_stats():
    cm = J.compile_graph(J.trace(_chain))
    x = torch.randn(2, 3)
    out = cm.run_tensors({"x": x})
    assert isinstance(cm.run({"x": x})["y"], list) and torch.allclose(out["y"], torch.relu(x) * 2 + 1, atol=1e-6)
    st = cm.stats()
    assert st.original_nodes == 5 and st.optimized_nodes <= 5 and 0.0 <= st.optimization_ratio() < 1.0 and st.passes >= 1
    assert cm.input_names() == ["x"] and cm.output_names() == ["y"]


def test_compile_fn_activations_and_matmul():
    def f(t):
        a, w = t.input("a", [3, 4]), t.input("w", [4, 2])
        t.output("y", a.matmul(w).gelu() if hasattr(a, "gelu") else a.matmul(w).relu())
    cm = J.compile_fn(f)
    a, w = torch.randn(3, 4), torch.randn(4, 2)
    y = cm.run_tensors({"a": a, "w": w})["y"]
    ref = torch.nn.functional.gelu(a @ w, approximate="tanh")
    assert torch.allclose(y, ref, atol=1e-4) or torch.allclose(y, torch.nn.functional.gelu(a @ w), atol=1e-4)


def test_compile_config_builder_and_enums():
    c = J.CompileConfig.new().mode(J.Mode.MaxAutotune).fullgraph(True).dynamic(False)
    assert {m.name for m in J.Mode} == {"Default", "ReduceOverhead", "MaxAutotune"}
    assert {b.name for b in J.Backend} == {"Default", "Interpreter", "Cuda"}
    cm = J.compile_graph_with_config(J.trace(_chain), c)
    assert cm.is_compiled()
    off = J.compile_graph_with_config(J.trace(_chain), J.CompileConfig.new().disable(True))
    x = torch.randn(2, 3)
    assert torch.allclose(off.run_tensors({"x": x})["y"], cm.run_tensors({"x": x})["y"])


# --------------------------------------------------------------------------------- optimisations
def test_dead_code_elimination_drops_unused_nodes():
    def f(t):
        x = t.input("x", [4])
        x.exp().neg()                                   # never reaches an output
        t.output("y", x.relu())
    g = J.trace(f)
    opt = J.Optimizer([J.OptimizationPass.DeadCodeElimination]).optimize(g)
    assert opt.len() == 3 and {n.op.kind for n in opt.nodes} == {"Input", "Relu", "Output"}


def test_constant_folding_and_algebraic_simplification():
    def f(t):
        x = t.input("x", [4])
        c = t.constant(2.0).mul(t.constant(3.0))
        t.output("y", x.mul(c).add_scalar(0.0).mul_scalar(1.0))
    g = J.trace(f)
    Ps = J.OptimizationPass
    opt = J.Optimizer([Ps.ConstantFolding, Ps.AlgebraicSimplification, Ps.DeadCodeElimination]).optimize(g)
    assert opt.len() < g.len()
    x = torch.randn(4)
    assert torch.allclose(J.interpret(opt, {"x": x})["y"], x * 6, atol=1e-6)


def test_common_subexpressions_are_shared():
    def f(t):
        x = t.input("x", [4])
        t.output("y", x.exp().add(x.exp()))
    g = J.trace(f)
    opt = J.Optimizer([J.OptimizationPass.CommonSubexpressionElimination, J.OptimizationPass.DeadCodeElimination]).optimize(g)
    assert sum(1 for n in opt.nodes if n.op.kind == "Exp") == 1
    x = torch.randn(4)
    assert torch.allclose(J.interpret(opt, {"x": x})["y"], 2 * x.exp(), atol=1e-6)


# ------------------------------------------------------------------------------------------ cache
def test_graph_hash_depends_on_structure_only():
    a, b = J.trace(_chain), J.trace(_chain)
    assert J.FunctionCache.hash_graph(a) == J.FunctionCache.hash_graph(b)
    other = J.trace(lambda t: t.output("y", t.input("x", [2, 3]).relu()))
    assert J.FunctionCache.hash_graph(a) != J.FunctionCache.hash_graph(other)


def test_function_cache_insert_get_evict_and_stats():
    cache = J.FunctionCache(2)
    graphs = [J.trace(lambda t, k=k: t.output("y", t.input("x", [k + 1]).relu())) for k in range(3)]
    comp = J.JitCompiler.new()
    for g in graphs[:2]:
        cache.insert_for_graph(g, comp.compile(g))
    assert cache.len() == 2 and cache.get_by_graph(graphs[0]) is not None
    cache.insert_for_graph(graphs[2], comp.compile(graphs[2]))
    assert cache.len() == 2                                                   # the oldest entry made room
    st = cache.stats()
    assert st.entries == 2 and st.max_size == 2 and 0.99 <= st.utilization() <= 100.0
    cache.clear()
    assert cache.is_empty()


def test_compiler_caches_compiled_functions():
    comp = J.JitCompiler.new()
    f1, f2 = comp.compile(J.trace(_chain)), comp.compile(J.trace(_chain))
    assert comp.cache_stats().entries == 1
    x = torch.randn(2, 3)
    assert torch.allclose(f1.run_tensors({"x": x})["y"], f2.run_tensors({"x": x})["y"])
    comp.clear_cache()
    assert comp.cache_stats().entries == 0


def test_jit_shape_helpers_and_errors():
    s = J.Shape.new([2, 1, 4])
    assert s.numel() == 8 and s.ndim() == 3 and s.broadcast_compatible([3, 1]) and s.broadcast_shape([3, 1]) == (2, 3, 4)
    with pytest.raises(J.JitError):
        J.compile_graph(J.trace(_chain)).run({})


# ----------------------------------------------------------------------------------------- fusion
def test_fused_linear_variants_match_the_unfused_computation():
    w, b, x = torch.randn(4, 3), torch.randn(4), torch.randn(5, 3)
    assert torch.allclose(FU.fuse_linear(w, b)(x), x @ w.t() + b, atol=1e-5)
    assert torch.allclose(FU.fuse_linear(w, None, FU.Activation.Relu)(x), torch.relu(x @ w.t()), atol=1e-5)
    assert torch.allclose(FU.fuse_linear(w, b, FU.Activation.Sigmoid)(x), torch.sigmoid(x @ w.t() + b), atol=1e-5)
    assert torch.allclose(FU.fuse_linear(w, b, FU.Activation.Tanh)(x), torch.tanh(x @ w.t() + b), atol=1e-5)
    assert torch.allclose(FU.fuse_linear(w, b, FU.Activation.Silu)(x), torch.nn.functional.silu(x @ w.t() + b), atol=1e-5)
    fl = FU.FusedLinear.new(w, b, FU.Activation.Relu) if hasattr(FU.FusedLinear, "new") else FU.FusedLinear(w, b, FU.Activation.Relu)
    assert fl.num_ops() == 3 and "relu" in fl.name().lower() and fl.execute(x).shape == (5, 4)


def test_fused_elementwise_chains():
    x = torch.linspace(-2, 2, 9)
    chain = FU.fused_elementwise().mul(2.0).add(1.0).relu().build()
    assert torch.allclose(chain(x), torch.relu(2 * x + 1)) and chain.num_ops() == 3
    assert torch.allclose(FU.fused_elementwise().sigmoid().build()(x), torch.sigmoid(x))
    assert torch.allclose(FU.fused_elementwise().abs().sqrt().build()(x), x.abs().sqrt())
    assert torch.allclose(FU.fused_elementwise().clamp(-1.0, 1.0).square().neg().build()(x), -x.clamp(-1, 1) ** 2)
    assert torch.allclose(FU.fused_elementwise().leaky_relu(0.1).build()(x), torch.nn.functional.leaky_relu(x, 0.1))


def test_pattern_detection():
    O, Pt = FU.OpType, FU.FusionPattern
    assert FU.detect_patterns([O.MatMul, O.Add, O.Relu]) == [(Pt.MatMulBiasRelu, 0, 3)]
    assert FU.detect_patterns([O.MatMul, O.Add, O.Gelu])[0][0] == Pt.MatMulBiasGelu
    assert FU.detect_patterns([O.MatMul, O.Add, O.Softmax])[0] == (Pt.MatMulBias, 0, 2)
    assert FU.detect_patterns([O.Conv, O.BatchNorm, O.Relu])[0][0] == Pt.ConvBatchNormRelu
    assert FU.detect_patterns([O.Other, O.Add, O.Relu]) == [(Pt.AddRelu, 1, 2)]
    assert FU.detect_patterns([O.Exp, O.Sqrt, O.Tanh]) == [(Pt.ElementwiseChain, 0, 3)]
    assert FU.detect_patterns([O.Other, O.Other]) == []


def test_fusion_optimizer_statistics_and_configurations():
    O = FU.OpType
    ops = [O.MatMul, O.Add, O.Relu, O.Other, O.Exp, O.Log]
    opt = FU.FusionOptimizer.new()
    patterns = opt.analyze(ops)
    assert len(patterns) == 2
    st = opt.stats()
    assert (st.total_ops, st.fused_ops, st.patterns_found) == (6, 5, 2) and st.estimated_speedup > 1.0 and st.fusion_ratio() == pytest.approx(5 / 6)
    assert opt.optimization_stats.fusions_applied == 2 and opt.optimization_stats.ops_eliminated == 3
    opt.reset_stats()
    assert opt.stats().patterns_found == 0 and opt.optimization_stats.fusions_applied == 0
    none = FU.FusionOptimizer.with_config(FU.FusionConfig(fuse_elementwise=False, fuse_linear=False, fuse_conv=False))
    assert none.analyze(ops) == []
    cons = FU.FusionConfig.conservative()
    assert not cons.aggressive and FU.FusionConfig.aggressive_mode().aggressive
    assert FU.estimate_speedup(ops, patterns) > 1.0 and FU.estimate_speedup(ops, []) == 1.0


def test_conv_batchnorm_folding_preserves_the_output():
    torch.manual_seed(0)
    conv, bn = torch.nn.Conv2d(3, 4, 3, padding=1), torch.nn.BatchNorm2d(4)
    bn.running_mean.uniform_(-1, 1), bn.running_var.uniform_(0.5, 2.0), bn.weight.data.uniform_(0.5, 1.5), bn.bias.data.uniform_(-1, 1)
    bn.eval()
    x = torch.randn(2, 3, 6, 6)
    w, b = FU.fold_conv_bn(conv, bn)
    assert torch.allclose(torch.nn.functional.conv2d(x, w, b, padding=1), bn(conv(x)), atol=1e-5)


# --------------------------------------------------------------------------------------- profiler
def test_compute_profiler_times_and_counts_calls():
    c = P.ComputeProfiler()
    for _ in range(3):
        c.start("op")
        time.sleep(0.002)
        c.stop("op")
    st = c.get_stats("op")
    assert st.count == 3 and st.total_ns >= 3 * 1.5e6 and st.min_ns <= st.avg_ns() <= st.max_ns
    assert c.get_stats("missing") is None and c.total_time_ns() >= st.total_ns
    c.reset()
    assert c.get_stats("op") is None


def test_compute_profiler_nested_operations_and_ranking():
    c = P.ComputeProfiler()
    c.start("outer")
    c.start("inner")
    time.sleep(0.002)
    c.stop("inner")
    time.sleep(0.001)
    c.stop("outer")
    assert c.get_stats("outer").total_ns > c.get_stats("inner").total_ns
    assert [s.name for s in c.top_by_time(2)] == ["outer", "inner"]
    c.record("cheap", 10.0)
    c.record("cheap", 10.0)
    assert c.top_by_calls(1)[0].name == "cheap"


def test_throughput_figures_from_flops_and_bytes():
    c = P.ComputeProfiler()
    c.start_with_flops("gemm", 2e9)
    time.sleep(0.002)
    c.stop("gemm")
    assert 0 < c.get_stats("gemm").gflops() < 1000
    c.start_with_bytes("copy", 1e9)
    time.sleep(0.002)
    c.stop("copy")
    assert 0 < c.get_stats("copy").gbps() < 500


def test_duration_and_byte_formatting():
    assert P.format_duration(500) == "500 ns" or "ns" in P.format_duration(500)
    assert "us" in P.format_duration(5_000) or "µs" in P.format_duration(5_000)
    assert "ms" in P.format_duration(5_000_000) and P.format_duration(2_500_000_000).endswith("s")
    assert P.format_bytes(512) == "512 B" and P.format_bytes(2048).startswith("2.00 K") and "M" in P.format_bytes(5 * 1024 ** 2)
    assert "G" in P.format_bytes(3 * 1024 ** 3)


def test_memory_profiler_tracks_usage_peak_and_leaks():
    m = P.MemoryProfiler()
    m.record_alloc("a", 1000)
    m.record_alloc("b", 500)
    m.record_free("a", 1000)
    assert m.current_usage() == 500 and m.peak_usage() == 1500
    leaks = m.leaks()
    assert [(l.name, l.size) for l in leaks] == [("b", 500)]
    st = m.stats()
    assert st.allocation_count == 2 and st.deallocation_count == 1 and st.total_freed == 1000
    m.reset()
    assert m.current_usage() == 0 and m.leaks() == []


def test_timeline_records_filters_and_caps_events():
    t = P.TimelineProfiler.with_capacity(4)
    t.record("load", P.EventType.Start)
    t.record("load", P.EventType.End)
    t.record_with_metadata("mark", P.EventType.Instant, "epoch=1")
    assert t.event_count() == 3 and len(t.events_by_name("load")) == 2 and len(t.events_by_type(P.EventType.Instant)) == 1
    assert t.events_by_name("mark")[0].metadata == "epoch=1" and t.duration("load") >= 0
    for i in range(5):
        t.record(f"x{i}", P.EventType.Instant)
    assert t.event_count() == 4                                               # capacity
    doc = json.loads(t.to_json()) if isinstance(t.to_json(), str) else t.to_json()
    assert isinstance(doc, (list, dict))
    t.reset()
    assert t.event_count() == 0


def test_profiler_facade_guard_enable_and_reset():
    p = P.Profiler.new()
    with p.scope("step"):
        time.sleep(0.001)
    p.start("io")
    p.stop("io")
    p.record_alloc("buf", 4096)
    assert p.total_time("step") > 0 and p.avg_time("step") > 0 and p.total_time("none") == 0 and p.peak_memory() == 4096 and p.current_memory() == 4096
    p.record_free("buf", 4096)
    assert p.current_memory() == 0
    p.set_enabled(False)
    p.start("ignored")
    p.stop("ignored")
    assert not p.is_enabled() and p.compute.get_stats("ignored") is None
    p.enable()
    p.reset()
    assert p.total_time("step") == 0 and p.peak_memory() == 0


def test_reports_in_every_format():
    p = P.Profiler.new()
    with p.scope("forward"):
        time.sleep(0.001)
    p.record_alloc("acts", 1 << 20)
    r = p.report()
    text, md, html_, js = r.format(P.ReportFormat.Text), r.format(P.ReportFormat.Markdown), r.format(P.ReportFormat.Html), r.format(P.ReportFormat.Json)
    assert "forward" in text and "|" in md and "forward" in md and "<html" in html_.lower() and "forward" in html_
    doc = json.loads(js)
    assert any("forward" in json.dumps(v) for v in doc.values())
    assert r.compute.operation_count == 1 and r.memory.peak_usage == 1 << 20


def test_bottleneck_analysis_finds_slow_operations_hotspots_and_leaks():
    p = P.Profiler.new()
    p.start("slow")
    time.sleep(0.01)
    p.stop("slow")
    p.start("fast")
    p.stop("fast")
    p.record_alloc("big", 10 << 20)
    p.record_alloc("small", 1 << 10)
    found = p.analyze_bottlenecks()
    kinds = {(b.bottleneck_type() if callable(getattr(b, "bottleneck_type", None)) else b.kind, b.name) for b in found}
    assert (P.BottleneckType.SlowOperation, "slow") in kinds
    assert any(k == P.BottleneckType.MemoryHotspot and n == "big" for k, n in kinds)
    assert any(k == P.BottleneckType.MemoryLeak for k, _ in kinds)
    assert all(b.suggestion and b.description and isinstance(b.severity, P.Severity) for b in found)
    assert "slow" in P.BottleneckAnalyzer.new().summary(p)
    assert P.BottleneckAnalyzer.new().summary(P.Profiler.new()) == "No bottlenecks detected."


# ----------------------------------------------------------------------------------- quantisation
@pytest.mark.parametrize("qt,tol", [(Q.QuantType.Q8_0, 0.02), (Q.QuantType.Q4_0, 0.2), (Q.QuantType.Q4_1, 0.15),
                                    (Q.QuantType.Q5_0, 0.1), (Q.QuantType.Q5_1, 0.08), (Q.QuantType.Q4_K, 0.15),
                                    (Q.QuantType.F16, 2e-3), (Q.QuantType.BF16, 2e-2), (Q.QuantType.F32, 0.0)])
def test_quantise_dequantise_round_trip_error(qt, tol):
    torch.manual_seed(0)
    x = torch.randn(4, 256)
    q = Q.quantize_tensor(x, qt)
    y = Q.dequantize_tensor(q)
    assert y.shape == x.shape and float((x - y).abs().max()) <= tol * float(x.abs().max()) + 1e-7
    assert q.numel() == x.numel() and q.size_bytes() == x.numel() // qt.block_size() * qt.bytes_per_block()


def test_quant_type_properties():
    T = Q.QuantType
    assert (T.Q8_0.block_size(), T.Q8_0.bytes_per_block()) == (32, 34) and (T.Q4_0.block_size(), T.Q4_0.bytes_per_block()) == (32, 18)
    assert T.Q4_1.bytes_per_block() == 20 and T.Q4_K.block_size() == 256 and T.Q4_K.bytes_per_block() == 144
    assert T.F32.block_size() == 1 and T.F16.bytes_per_block() == 2 and not T.F16.is_block_quantized() and T.Q5_0.is_block_quantized()
    assert T.Q8_0.bits_per_value() == 8.5 and T.Q4_0.bits_per_value() == 4.5 and T.Q4_0.nominal_bits() == 4
    assert T.Q4_0.compression_ratio() == 8.0 and T.Q8_0.compression_ratio() == 4.0 and T("q8_0") is T.Q8_0
    for t in T:
        assert T.from_ggml_type(t.ggml_type()) is t


def test_q4_pack_unpack_and_q8_block():
    vals = [-8, -1, 0, 7] * 8
    b = Q.Q4Block.new(0.5, Q.Q4Block.pack(vals)) if hasattr(Q.Q4Block, "pack") else None
    assert b.unpack() == vals and b.dequantize() == [v * 0.5 for v in vals]
    assert Q.Q4Block.from_bytes(b.to_bytes()).unpack() == vals and len(b.to_bytes()) == 18
    q8 = Q.Q8Block.new(0.25, list(range(-16, 16)))
    assert q8.dequantize()[0] == -4.0 and len(q8.to_bytes()) == 34 and Q.Q8Block.from_bytes(q8.to_bytes()).data == q8.data


def test_quantised_tensor_blocks_and_compression():
    x = torch.randn(2, 64)
    q = Q.quantize_tensor(x, Q.QuantType.Q8_0)
    assert q.num_blocks() == 4 and len(list(q.blocks())) == 4 and q.compression_ratio() == pytest.approx(32 * 4 / 34)
    blk = q.block(1)
    assert torch.allclose(torch.tensor(blk.dequantize()), x.flatten()[32:64], atol=0.02 * float(x.abs().max()))
    assert Q.dequantize_block(blk.to_bytes(), Q.QuantType.Q8_0) == blk.dequantize()


def test_calibration_statistics_scales_and_methods():
    x = torch.tensor([-2.0, -1.0, 0.0, 1.0, 4.0])
    c = Q.calibrate(x)
    assert (c.min, c.max) == (-2.0, 4.0) and c.mean == pytest.approx(0.4) and c.count == 5 and c.dynamic_range() == 6.0
    assert c.symmetric_scale(Q.QuantType.Q8_0) == pytest.approx(4.0 / 127) and c.symmetric_scale(Q.QuantType.Q4_0) == pytest.approx(4.0 / 7)
    scale, zero = c.asymmetric_scale(Q.QuantType.Q8_0)
    assert scale == pytest.approx(6.0 / 255) and zero == -2.0
    c.update(torch.tensor([10.0]))
    assert c.max == 10.0 and c.count == 6
    big = torch.cat([torch.randn(10000), torch.tensor([100.0])])
    assert Q.calibrate(big, Q.CalibrationMethod.Percentile).max < 100.0 <= Q.calibrate(big, Q.CalibrationMethod.MinMax).max
    assert Q.calibrate(big, Q.CalibrationMethod.MeanStd).max < 100.0
    assert Q.calibrate_batch([x, x * 2]).max == 8.0


def test_quantisation_error_and_model_quantisation():
    x = torch.randn(8, 128)
    y8, y4 = (Q.dequantize_tensor(Q.quantize_tensor(x, t)) for t in (Q.QuantType.Q8_0, Q.QuantType.Q4_0))
    assert 0 < Q.compute_quantization_error(x, y8) < Q.compute_quantization_error(x, y4)
    st = Q.compute_quantization_stats(x, y4, Q.QuantType.Q4_0)
    assert st.max_error >= st.mean_error > 0 and st.rmse > 0 and st.compression_ratio == 8.0
    out = Q.quantize_model({"big": torch.randn(64, 64), "tiny": torch.randn(8)}, Q.QuantType.Q8_0)
    assert out["big"].quant_type is Q.QuantType.Q8_0 and out["tiny"].quant_type is Q.QuantType.F32            # small tensors stay exact
