"""LLM families (GPT-2, LLaMA, BERT, Mistral, Phi) on tiny configurations, KV-cache generation,
JIT tracing / optimisation / interpretation, fusion, profiler, text and audio utilities, hub, the
serving stack on the CPU (paged KV cache, continuous batching, HTTP endpoints) and the trainer."""
import json
import threading
import urllib.request

import pytest
import torch

from axonml_b200 import audio, fusion, hub, jit, llm, nn, optim, profile, server, text, trainer, vision
from axonml_b200.quant import QuantType


def test_gpt2_and_llama_tiny_train_step_reduces_loss():
    torch.manual_seed(0)
    for model in (llm.GPT2LMHead(llm.GPT2Config.tiny()), llm.LLaMAForCausalLM(llm.LLaMAConfig.tiny())):
        ids = torch.randint(0, 100, (2, 16))
        opt = optim.AdamW(list(model.parameters()), 3e-3)
        first = None
        for _ in range(8):
            opt.zero_grad()
            loss, logits = model.forward_with_loss(ids)
            loss.backward()
            opt.step()
            first = first if first is not None else float(loss)
        assert logits.shape[:2] == (2, 16)
        assert float(loss) < first


def test_llama_kv_cache_generation_matches_full_forward():
    torch.manual_seed(0)
    model = llm.LLaMAForCausalLM(llm.LLaMAConfig.tiny()).eval()
    ids = torch.randint(0, 100, (1, 6))
    out = model.generate(ids, max_new_tokens=5)
    out = out if torch.is_tensor(out) else torch.tensor(out)
    assert out.shape[-1] == 11
    # greedy continuation token by token without a cache
    cur = ids.clone()
    with torch.no_grad():
        for _ in range(5):
            nxt = model(cur)[:, -1].argmax(-1, keepdim=True)
            cur = torch.cat([cur, nxt], 1)
    assert torch.equal(out.view(-1), cur.view(-1))


def test_bert_mistral_phi_forward_shapes():
    torch.manual_seed(0)
    b = llm.BertForSequenceClassification(llm.BertConfig.tiny(), 3).eval()
    ids = torch.randint(0, 100, (2, 10))
    out = b(ids)
    out = out[0] if isinstance(out, tuple) else out
    assert out.shape == (2, 3)
    for cls, cfg in ((llm.MistralForCausalLM, llm.MistralConfig.tiny() if hasattr(llm.MistralConfig, "tiny") else None),
                     (llm.PhiForCausalLM, llm.PhiConfig.tiny())):
        if cfg is None:
            continue
        m = cls(cfg).eval()
        y = m(torch.randint(0, 100, (1, 8)))
        y = y[0] if isinstance(y, tuple) else y
        assert y.shape[:2] == (1, 8)


def test_hf_weight_mapping_names():
    sd = {"wte.weight": torch.zeros(2, 2), "h.0.attn.c_attn.weight": torch.zeros(2, 6)}
    mapped = llm.map_gpt2_weights(sd)
    assert len(mapped) == 2


def test_jit_trace_optimize_interpret_and_codegen():
    def f(tr):
        a, b = tr.input("a", [4]), tr.input("b", [4])
        y = a.add(b).mul_scalar(2.0).relu()
        return tr.output("y", y)
    g = jit.trace(f)
    assert len(g.input_names()) == 2 and not g.is_empty()
    a, b = torch.tensor([1.0, -2.0, 3.0, 0.5]), torch.tensor([1.0, 1.0, -5.0, 0.5])
    out = jit.interpret(g, {"a": a, "b": b})
    assert torch.allclose(out["y"], ((a + b) * 2).relu())
    cm = jit.compile_graph(g)
    got = cm.run_tensors({"a": a, "b": b})
    assert torch.allclose(got["y"], ((a + b) * 2).relu())
    src = jit.generate_cuda(g)
    src = src if isinstance(src, str) else src[0]
    assert "__global__" in src


def test_jit_lowering_plan_for_reductions_and_broadcast_is_generated_without_a_gpu():
    """The multi-kernel lowering is a source-to-source step: it can be checked here for structure
    (one kernel per materialised value, the matrix product left to the GEMM), and the interpreter
    evaluates the same graph, reshape and broadcast included."""
    from axonml_b200.jit import lower

    def f(tr):
        x, b = tr.input("x", [8, 12]), tr.input("b", [12])
        z = x.add(b)
        p = z.sub(z.max_axis(1, True)).exp()
        p = p.div(p.sum_axis(1, True))
        tr.output("p", p)
        tr.output("pt", p.transpose(0, 1).reshape([12, 8]))
        tr.output("g", p.matmul(p.transpose(0, 1)))
        tr.output("big", b.broadcast([8, 12]))
    g = jit.trace(f)
    assert lower.lowerable(g)
    plan = lower.Plan(g)
    kinds = [s["kind"] for s in plan.steps]
    assert kinds.count("matmul") == 1 and kinds.count("kernel") >= 4
    assert plan.source.count("__global__") == kinds.count("kernel")
    x, b = torch.randn(8, 12), torch.randn(12)
    out = jit.interpret(g, {"x": x, "b": b})
    ref = torch.softmax(x + b, -1)
    assert torch.allclose(out["p"], ref, atol=1e-6) and torch.allclose(out["pt"], ref.t(), atol=1e-6)
    assert torch.allclose(out["g"], ref @ ref.t(), atol=1e-6) and torch.equal(out["big"], b.expand(8, 12))


def test_fusion_linear_and_elementwise_and_conv_bn_fold():
    torch.manual_seed(0)
    w, b = torch.randn(3, 4), torch.randn(3)
    fl = fusion.fuse_linear(w, b, fusion.Activation.ReLU if hasattr(fusion.Activation, "ReLU") else list(fusion.Activation)[1])
    x = torch.randn(2, 4)
    assert fl.execute(x).shape == (2, 3)
    fe = fusion.FusedElementwiseBuilder().mul(2.0).add(1.0).relu().build()
    assert torch.allclose(fe.execute(torch.tensor([-3.0, 1.0])), torch.tensor([0.0, 3.0]))
    assert fe.num_ops() == 3
    conv, bn = nn.Conv2d(2, 3, 3, padding=1), nn.BatchNorm2d(3)
    bn.eval()
    with torch.no_grad():
        bn.running_mean.uniform_(-1, 1); bn.running_var.uniform_(0.5, 2.0)
        bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-1, 1)
    fw, fb = fusion.fold_conv_bn(conv, bn)         # folded (weight, bias)
    xx = torch.randn(1, 2, 5, 5)
    assert torch.allclose(torch.nn.functional.conv2d(xx, fw, fb, 1, 1), bn(conv(xx)), atol=1e-5)


def test_profiler_report_and_chrome_trace(tmp_path):
    p = profile.Profiler()
    p.enable()
    with p.scope("matmul"):
        torch.randn(64, 64) @ torch.randn(64, 64)
    with p.scope("matmul"):
        torch.randn(64, 64) @ torch.randn(64, 64)
    rep = p.report()
    ops = {(o["name"] if isinstance(o, dict) else o.name): o for o in rep.operations}
    assert "matmul" in ops
    assert "matmul" in rep.to_markdown() and "matmul" in rep.to_json()
    tl = profile.TimelineProfiler()
    tl.begin("step"); tl.end("step")
    out = tmp_path / "trace.json"
    tl.export_chrome_trace(str(out))
    ev = json.load(open(out))
    ev = ev["traceEvents"] if isinstance(ev, dict) else ev
    assert any(e.get("name") == "step" for e in ev)


def test_text_and_audio_utilities():
    tok = text.BasicBPETokenizer()
    tok.train("low lower lowest low low", 20) if "num_merges" not in str(tok.train.__code__.co_varnames) else tok.train("low lower lowest", 20)
    assert len(tok.tokenize("lower")) >= 1
    v = text.Vocab.from_text("the cat sat on the mat")
    ids = v.encode(["the", "cat"]) if not isinstance(v.encode("the cat"), list) or len(v.encode("the cat")) != 2 else v.encode("the cat")
    dec = v.decode(ids)
    assert (dec.split() if isinstance(dec, str) else list(dec)) == ["the", "cat"]
    assert text.CharTokenizer().tokenize("ab c") == ["a", "b", " ", "c"]
    ds = text.LanguageModelDataset(list(range(50)), 8)
    x, y = ds.get(0)
    assert torch.equal(x[1:], y[:-1])
    wave = torch.sin(torch.linspace(0, 200.0, 16000))
    mel = audio.MelSpectrogram(16000, 400, 160, 40).apply(wave)
    assert mel.shape[0] == 40 or mel.shape[-2] == 40 or mel.shape[-1] == 40
    assert audio.MFCC(16000, 13, 40).apply(wave).numel() > 0
    assert abs(audio.Resample(16000, 8000).apply(wave).numel() - 8000) <= 2
    a, lab = audio.SyntheticCommandDataset(4).get(0)
    assert a.numel() == 16000


def test_hub_registry():
    names = [m.name for m in hub.list_all_models()]
    assert "resnet18" in names
    info = hub.get_model_info("resnet18")
    assert 11_000_000 < info.num_parameters < 12_500_000
    assert any("gpt" in m.name.lower() for m in hub.search_models("gpt"))


def test_vision_models_forward():
    assert vision.LeNet.new()(torch.randn(2, 1, 28, 28)).shape == (2, 10)
    r = vision.ResNet.resnet18(10).eval()
    assert r(torch.randn(1, 3, 64, 64)).shape == (1, 10)
    assert sum(p.numel() for p in vision.ResNet.resnet18(1000).parameters()) == 11_689_512


def test_paged_kv_cache_bookkeeping():
    c = server.PagedKVCache(2, 8, 4, 1, 8, 4, 4, "cpu", torch.float32)
    s0, s1 = c.allocate_seq(), c.allocate_seq()
    c.reserve(s0, 9)                      # 3 pages
    c.reserve(s1, 4)                      # 1 page
    assert c.pages_free() == 4 and abs(c.occupancy() - 0.5) < 1e-9
    assert not c.can_admit(17) and c.can_admit(16)
    with pytest.raises(server.OutOfPages):
        c.reserve(s1, 4 * 6)
    c.free_seq(s0)
    assert c.pages_free() == 7


def test_engine_continuous_batching_matches_sequential_decode_cpu():
    torch.manual_seed(0)
    cfg = llm.LLaMAConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                          num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=128)
    model = server.QuantizedLlama.from_random(cfg, None, device="cpu", std=0.2, proj_type=QuantType.Q8_0)
    prompts = [[1, 2, 3, 4], [9, 8, 7, 6], [5, 5, 5, 5]]
    together = server.LLMEngine(model, max_batch=4, max_context=32, page_size=4).generate(prompts, 5)
    alone = [server.LLMEngine(model, max_batch=4, max_context=32, page_size=4).generate([p], 5)[0] for p in prompts]
    assert together == alone
    st = server.LLMEngine(model, max_batch=4, max_context=32, page_size=4)
    st.generate(prompts, 3)
    s = st.stats()
    assert s["requests"] == 3 and s["kv_page_occupancy"] == 0.0 and s["ttft_p50_s"] is not None


def test_http_server_endpoints():
    from axonml_b200.serialize.state_dict import StateDict
    torch.manual_seed(0)
    m = nn.Sequential().add(nn.Linear(4, 8)).add(nn.ReLU()).add(nn.Linear(8, 2))
    inf = server.InferenceServer()
    inf.register("mlp", server.build_model_from_state_dict(StateDict.from_module(m)))
    srv = server.AxonmlHTTPServer("127.0.0.1", 0, inf).start()
    try:
        port = srv.port if hasattr(srv, "port") else srv.httpd.server_address[1]
        base = f"http://127.0.0.1:{port}"
        assert json.load(urllib.request.urlopen(base + "/health"))["status"] == "healthy"
        req = urllib.request.Request(base + "/batch", method="POST", headers={"Content-Type": "application/json"},
                                     data=json.dumps({"model": "mlp", "inputs": [[1.0, 2.0, 3.0, 4.0]]}).encode())
        body = json.load(urllib.request.urlopen(req))
        got = torch.tensor(body["outputs"])
        req = urllib.request.Request(base + "/api/inference/predict/mlp", method="POST",
                                     data=json.dumps({"input": [1.0, 2.0, 3.0, 4.0]}).encode())
        one = json.load(urllib.request.urlopen(req))
        assert torch.allclose(torch.tensor(one["output"]).view(-1), got.view(-1), atol=1e-6) and one["latency_ms"] >= 0
        assert torch.allclose(got.view(-1), m(torch.tensor([[1.0, 2.0, 3.0, 4.0]])).view(-1), atol=1e-5)
        prom = urllib.request.urlopen(base + "/metrics").read().decode()
        assert "axonml" in prom
    finally:
        srv.stop()


def test_trainer_fit_with_early_stopping():
    torch.manual_seed(0)
    from axonml_b200 import data
    X = torch.randn(128, 4)
    Y = (X.sum(-1) > 0).long()
    loader = data.DataLoader(data.TensorDataset(X, Y), 32)
    model = nn.Sequential().add(nn.Linear(4, 16)).add(nn.ReLU()).add(nn.Linear(16, 2))
    cfg = trainer.TrainingConfig.new().epochs(15).learning_rate(0.01)
    t = trainer.Trainer(model, optim.Adam(list(model.parameters()), 0.01), nn.CrossEntropyLoss(), cfg,
                        callbacks=[trainer.EarlyStopping(3)])
    hist = t.fit(loader, loader)
    metrics = t.evaluate(loader)
    acc = metrics.accuracy if hasattr(metrics, "accuracy") else metrics["accuracy"]
    assert acc > 0.85


def test_jit_errors_node_ids_and_shapes():
    from axonml_b200.jit import error as JE
    g = jit.trace(lambda t: t.output("y", t.input("x", [2, 3]).relu().mul_scalar(2.0)))
    assert all(isinstance(n.id, jit.NodeId) and n.id.index() == i for i, n in enumerate(g.nodes)) and repr(g.nodes[1].id) == "%1"
    assert isinstance(g.nodes[0].shape, jit.Shape) and g.nodes[0].shape.numel() == 6 and g.nodes[0].shape.ndim() == 2
    f = jit.JitCompiler().compile(g)
    assert f.run([("x", [-1.0, 2.0, -3.0, 4.0, 0.5, -0.5])]) == [0.0, 4.0, 0.0, 8.0, 1.0, 0.0]
    with pytest.raises(JE.InputNotFound) as e:
        f.run([("z", [1.0] * 6)])
    assert str(e.value) == "Input not found: z" and isinstance(e.value, (jit.JitError, KeyError))
    with pytest.raises(JE.InputNotFound):
        f.run([])
    with pytest.raises(JE.ShapeMismatch) as e:
        f.run([("x", [1.0, 2.0])])
    assert e.value.expected == [2, 3] and e.value.found == [2]
    with pytest.raises(JE.UnsupportedOp) as e:
        jit.Op.make("Conv3d")
    assert isinstance(e.value, NotImplementedError) and "Conv3d" in str(e.value)
    bad = jit.Graph()
    bad.add_node(jit.Op.make("Neg", [3]), jit.DataType.F32, [2])
    with pytest.raises(JE.InvalidGraph):
        bad.validate()
    s = jit.Shape.new([4, 1, 3])
    assert s.dims() == (4, 1, 3) and s.broadcast_compatible([5, 3]) and not s.broadcast_compatible([2, 3, 3])
    assert s.broadcast_shape([5, 1]) == (4, 5, 3) and s.broadcast_shape([2, 2, 2]) is None and jit.Shape().numel() == 1
    for cls in (JE.TypeMismatch("f32", "i64"), JE.CodegenError("x"), JE.JitRuntimeError("x"), JE.OutputNotFound("y"), JE.CompilationFailed("x")):
        assert isinstance(cls, jit.JitError)
    assert str(JE.TypeMismatch("f32", "i64")) == "Type mismatch: expected f32, found i64"


def test_fusion_errors_and_convenience_constructors():
    w, b = torch.randn(4, 3), torch.randn(4)
    x = torch.randn(5, 3)
    assert torch.allclose(fusion.fuse_matmul_bias_relu(w, b)(x), torch.relu(x @ w.t() + b), atol=1e-5)
    assert torch.allclose(fusion.fuse_matmul_bias(w, b)(x), x @ w.t() + b, atol=1e-5)
    assert torch.allclose(fusion.fuse_matmul_bias_gelu(w, b)(x), torch.nn.functional.gelu(x @ w.t() + b, approximate="tanh"), atol=1e-5)
    with pytest.raises(fusion.FusionError, match=r"expected \[4\], got \[3\]"):
        fusion.fuse_matmul_bias_relu(w, torch.randn(3))
    with pytest.raises(fusion.FusionError, match=r"expected \[3\], got \[7\]"):
        fusion.fuse_matmul_bias(w, b)(torch.randn(2, 7))
    with pytest.raises(fusion.FusionError, match="Invalid fusion configuration"):
        fusion.FusedLinear(torch.randn(4), None)
    with pytest.raises(fusion.FusionError, match="unknown activation"):
        fusion.FusedLinear(w, b, "softsign")
    E = fusion.ElementwiseOp
    chain = fusion.fuse_elementwise([(E.Mul, 2.0), (E.Add, -1.0), E.Relu, (E.Clamp, 0.0, 3.0)])
    v = torch.linspace(-2, 4, 13)
    assert chain.num_ops() == 4 and torch.allclose(chain(v), torch.clamp(torch.relu(v * 2 - 1), 0, 3), atol=1e-6)
    assert torch.allclose(fusion.fused_add_relu(0.5)(v), torch.relu(v + 0.5)) and torch.allclose(fusion.fused_mul_add(3.0, 1.0)(v), v * 3 + 1)
    assert torch.allclose(fusion.fused_scale_bias_relu(-1.0, 1.0)(v), torch.relu(1 - v))
    with pytest.raises(fusion.FusionError):
        fusion.fuse_elementwise(["relu"])


def test_profiler_records_stats_and_events():
    m = profile.MemoryProfiler()
    m.record_alloc("weights", 4096)
    m.record_alloc("acts", 1024)
    m.record_alloc("acts", 1024)
    m.record_free("acts", 1024)
    st = m.stats()
    assert isinstance(st, profile.MemoryStats) and (st.current_usage, st.peak_usage, st.total_allocated, st.total_freed) == (5120, 6144, 6144, 1024)
    assert (st.allocation_count, st.deallocation_count) == (3, 1) and st.per_name_usage == {"weights": 4096, "acts": 1024}
    leaks = m.leaks()
    assert [(r.name, r.size, r.freed) for r in leaks] == [("weights", 4096, False), ("acts", 1024, False)]
    assert all(isinstance(r, profile.AllocationRecord) for r in leaks) and leaks[0].timestamp <= leaks[1].timestamp
    assert sum(r.freed for r in m.records) == 1 and m.current_usage() == 5120 and m.peak_usage() == 6144
    assert profile.format_bytes(1536) == "1.50 KB" and profile.MemoryProfiler.format_bytes(3 << 30) == "3.00 GB" and profile.format_bytes(12) == "12 B"
    m.reset()
    assert m.stats() == profile.MemoryStats()

    c = profile.ComputeProfiler()
    c.start_with_flops("gemm", 2e9)
    assert [(op.name, op.flops) for op in c.active()] == [("gemm", 2e9)] and isinstance(c.active()[0], profile.ProfiledOp)
    c.stop("gemm")
    c.start_with_bytes("copy", 1 << 20); c.stop("copy")
    c.record("gemm", 1e6, flops=2e9)
    g = c.get_stats("gemm")
    assert g.count == 2 and g.flops == 4e9 and g.gflops() > 0 and c.get_stats("copy").bytes == 1 << 20 and c.get_stats("nope") is None
    assert c.total_time("gemm") == g.total_time() > 0 and c.avg_time("gemm") == pytest.approx(g.total_time() / 2) and c.total_time("nope") == 0.0
    assert g.min_time() <= g.avg_time() <= g.max_time() and not c.active()
    assert [s.name for s in c.top_by_calls(1)] == ["gemm"] and set(c.all_stats()) == {"gemm", "copy"}
    with pytest.raises(profile.ProfileError, match="Operation not found: nope"):
        c.require_stats("nope")
    assert profile.format_duration(1.5e6) == "1.500 ms" and profile.format_duration(2.5e9) == "2.500 s" and profile.format_duration(750) == "750 ns"

    t = profile.TimelineProfiler.with_capacity(6)
    t.start("step"); t.instant("mark"); t.record_with_metadata("buf", profile.EventType.Alloc, "4096"); t.end("step")
    t.record("note", profile.EventType.Custom)
    assert t.event_count() == 5 and [e.event_type for e in t.events] == [profile.EventType.Start, profile.EventType.Instant,
                                                                         profile.EventType.Alloc, profile.EventType.End, profile.EventType.Custom]
    assert len(t.events_by_name("step")) == 2 and t.events_by_type(profile.EventType.Alloc)[0].metadata == "4096"
    assert 0 <= t.duration("step") <= t.total_duration() and t.duration("mark") is None and t.duration("absent") is None
    assert all(isinstance(e, profile.Event) and e.thread_id is not None for e in t.events)
    t.instant("six"); t.instant("seven")
    assert t.event_count() == 6 and t.dropped == 1                              # capacity reached
    trace = json.loads(t.to_chrome_trace())["traceEvents"]
    assert [e["ph"] for e in trace[:4]] == ["B", "i", "i", "E"] and trace[2]["args"] == {"type": "Alloc", "metadata": "4096"}
    rows = json.loads(t.to_json())
    assert rows[0]["event_type"] == "Start" and rows[2]["metadata"] == "4096"
    with pytest.raises(profile.ProfileError):
        t.export_chrome_trace("/nonexistent-dir/trace.json")

    p = profile.Profiler()
    p.record_alloc("kv", 100); p.record_free("kv", 100)
    assert [e.event_type for e in p.timeline.events] == [profile.EventType.Alloc, profile.EventType.Free] and not p.memory.leaks()
    p.disable()
    p.record_alloc("kv", 100)
    assert p.memory.stats().allocation_count == 1


def test_quant_block_types_agree_with_the_codec():
    from axonml_b200 import quant as Q
    torch.manual_seed(0)
    w = torch.randn(2, 64)
    assert Q.DEFAULT_BLOCK_SIZE == 32 and Q.MAX_BLOCK_SIZE == 256 == Q.QuantType.Q4_K.block_size()
    q8 = Q.quantize_tensor(w, Q.QuantType.Q8_0)
    raw = q8.block(1).to_bytes()
    b8 = Q.Q8Block.from_bytes(raw)
    assert b8.to_bytes() == raw and b8.scale == q8.block(1).scale and len(b8.data) == 32
    assert torch.allclose(torch.tensor(b8.dequantize()), Q.dequantize_tensor(q8).flatten()[32:64])
    assert b8.as_block().quant_type is Q.QuantType.Q8_0 and Q.Q8Block.from_bytes(raw[:10]) is None
    # the reference's nibble order: value 2i in the low and 2i+1 in the high half of byte i
    vals = [(i % 16) - 8 for i in range(32)]
    packed = Q.Q4Block.pack(vals)
    assert packed[0] == (0 | (1 << 4)) and packed[1] == (2 | (3 << 4))
    b4 = Q.Q4Block.new(0.25, packed)
    assert b4.unpack() == vals and Q.Q4Block.from_bytes(b4.to_bytes()) == b4 and len(b4.to_bytes()) == 18
    q4 = Q.quantize_tensor(w, Q.QuantType.Q4_0, layout="adjacent")
    blk = Q.Q4Block.from_bytes(q4.block(3).to_bytes())
    assert torch.allclose(torch.tensor(blk.dequantize()), Q.dequantize_tensor(q4).flatten()[96:128])
    assert blk.as_block().dequantize() == pytest.approx(blk.dequantize())
    q41 = Q.quantize_tensor(w, Q.QuantType.Q4_1, layout="adjacent")
    b41 = Q.Q4_1Block.from_bytes(q41.block(0).to_bytes())
    assert len(b41.to_bytes()) == 20 and all(0 <= v <= 15 for v in b41.unpack())
    assert torch.allclose(torch.tensor(b41.dequantize()), Q.dequantize_tensor(q41).flatten()[:32], atol=1e-6)
    assert b41.min == q41.block(0).min and [b.quant_type for b in q41.blocks()] == [Q.QuantType.Q4_1] * 4
    with pytest.raises(Q.QuantError):
        Q.Q4Block.pack([9] * 32)
    with pytest.raises(Q.QuantError):
        Q.Q8Block(1.0, [0] * 31)
    with pytest.raises(Q.QuantError):
        Q.QuantizedBlock(Q.QuantType.Q8_0, b"\x00" * 5)
    with pytest.raises(IndexError):
        q8.block(99)


def test_bottleneck_severities_summaries_and_guards():
    S, T = profile.Severity, profile.BottleneckType
    p = profile.Profiler()
    p.compute.record("attention", 55e6)
    p.compute.record("mlp", 30e6)
    p.compute.record("norm", 15e6, flops=1e3)                # 6.7e-5 GFLOPS: a throughput finding
    for _ in range(3):
        p.compute.record("tiny", 1.0)
    p.compute.stats["tiny"].count = 60_000
    p.memory.record_alloc("kv_cache", 700)
    p.memory.record_alloc("acts", 300)
    p.memory.record_free("acts", 300)
    found = profile.BottleneckAnalyzer().analyze(p)
    by = {(b.kind, b.name.split(",")[0]): b for b in found}
    assert by[(T.SlowOperation, "attention")].severity is S.Critical and by[(T.SlowOperation, "mlp")].severity is S.Medium
    assert (T.SlowOperation, "norm") not in by and by[(T.LowThroughput, "norm")].severity is S.Medium
    assert by[(T.HighCallCount, "tiny")].severity is S.Medium and by[(T.HighCallCount, "tiny")].metrics["calls"] == 60_000
    assert by[(T.MemoryHotspot, "kv_cache")].severity is S.High and by[(T.MemoryHotspot, "acts")].severity is S.Low
    leak = by[(T.MemoryLeak, "kv_cache")]
    assert leak.severity is S.Critical and leak.metrics["leaked_bytes"] == 700 and leak.bottleneck_type is T.MemoryLeak
    sev = [b.severity for b in found]
    assert sev == sorted(sev, reverse=True) and S.Low < S.Medium < S.High < S.Critical and float(S.High) == 0.75
    cfg = profile.AnalyzerConfig(slow_op_threshold_pct=60.0, high_call_threshold=100_000, memory_hotspot_threshold_pct=90.0, check_memory_leaks=False)
    assert {b.kind for b in profile.BottleneckAnalyzer.with_config(cfg).analyze(p)} == {T.LowThroughput}
    d = profile.AnalyzerConfig()
    assert (d.slow_op_threshold_pct, d.high_call_threshold, d.memory_hotspot_threshold_pct, d.min_gflops_threshold, d.check_memory_leaks) == (20.0, 10_000, 30.0, 1.0, True)
    assert "[CRITICAL] SlowOperation" in profile.BottleneckAnalyzer().summary(p) and profile.BottleneckAnalyzer().summary(profile.Profiler()) == "No bottlenecks detected."
    rep = p.report()
    assert isinstance(rep.memory, profile.MemorySummary) and (rep.memory.peak_usage, rep.memory.current_usage, rep.memory.allocation_count) == (1000, 700, 2)
    assert isinstance(rep.compute, profile.ComputeSummary) and rep.compute.operation_count == 4 and rep.compute.total_time_ns == 100_000_003
    top = rep.compute.top_operations[0]
    assert isinstance(top, profile.OperationSummary) and top.name == "attention" and top.time_percentage == pytest.approx(55.0, abs=1e-3)
    assert "[Critical] [slow_operation]" in rep.to_text() and '"severity": "Critical"' in rep.to_json()

    c = profile.ComputeProfiler()
    with profile.TimingGuard(c, "step"):
        assert [op.name for op in c.active()] == ["step"]
    g = profile.TimingGuard.new(c, "step")
    g.drop(); g.drop()
    assert c.get_stats("step").count == 2 and not c.active()
    gp = profile.global_profiler()
    before = gp.memory.stats().allocation_count
    profile.start("global-op"); profile.stop("global-op"); profile.record_alloc("g", 8); profile.record_free("g", 8)
    assert gp.compute.get_stats("global-op").count >= 1 and gp.memory.stats().allocation_count == before + 1

    opt = fusion.FusionOptimizer()
    O = fusion.OpType
    opt.analyze([O.MatMul, O.Add, O.Relu, O.Conv, O.BatchNorm, O.MatMul, O.Add, O.Relu])
    st = opt.optimization_stats
    P = fusion.FusionPattern
    assert isinstance(st, fusion.OptimizationStats) and st.fusions_applied == 3 and st.ops_eliminated == 5
    assert st.patterns == [[P.MatMulBiasRelu, 2], [P.ConvBatchNorm, 1]]
    assert st.estimated_speedup == pytest.approx(P.MatMulBiasRelu.estimated_speedup() ** 2 * P.ConvBatchNorm.estimated_speedup())


def test_text_and_audio_conveniences():
    assert text.WhitespaceTokenizer.lowercase().tokenize("Hello World") == ["hello", "world"] and text.WhitespaceTokenizer().tokenize("Hi There") == ["Hi", "There"]
    assert text.WordPunctTokenizer.lowercase().tokenize("Hi, You!") == ["hi", ",", "you", "!"]
    assert text.CharTokenizer.no_whitespace().tokenize("a b\tc") == ["a", "b", "c"]
    bpe = text.BasicBPETokenizer()
    bpe.train("low lower lowest low low", 6)
    gv = bpe.get_vocab()
    assert gv == sorted(gv) and all(isinstance(t, str) for t in gv) and set(bpe.tokenize("low")) <= set(gv)
    uni = text.UnigramTokenizer.from_tokens(["un", "break", "able"])
    assert uni.tokenize("unbreakable") == ["un", "break", "able"] and uni.vocab["un"] == 1.0
    v = text.Vocab.new()
    assert v.is_empty()
    v.add_special_tokens(["<s>", "</s>"])
    v.set_unk_token("<?>")
    v.set_pad_token("<_>")
    v.add_token("cat")
    assert v.tokens() == ["<s>", "</s>", "<?>", "<_>", "cat"] and not v.is_empty() and v.token_to_index("dog") == 2 and v.pad_index() == 3
    samples = [("the cat sat", 0), ("the dog sat", 1), ("the cat ran", 2)]
    ds = text.TextDataset.from_samples(samples, text.WhitespaceTokenizer(), min_freq=2, max_length=5)
    toks = ds.vocab.tokens()
    assert toks[5:] == ["the", "cat", "sat"] and (ds.num_classes(), ds.max_length(), ds.len()) == (3, 5, 3)        # by count, ties alphabetically
    x, y = ds.get(1)
    assert x.tolist() == [5, ds.vocab.unk_index, 7, 0, 0] and int(y) == 1
    lm = text.LanguageModelDataset.from_text("a b c d e f g h", text.Vocab.from_text("a b c d e f g h"), text.WhitespaceTokenizer(), 3)
    assert lm.vocab() is not None and text.LanguageModelDataset(list(range(9)), 4).vocab() is None
    s = text.SyntheticSentimentDataset.small()
    assert s.len() == 100 and s.get(0)[0].shape == (32,) and text.SyntheticSentimentDataset.test().len() == 2000
    c = audio.SyntheticCommandDataset.small()
    assert (c.len(), c.sample_rate(), c.num_classes(), c.get(0)[0].numel()) == (100, 16000, 10, 8000)
    assert audio.SyntheticCommandDataset.large().num_classes() == 35 and audio.SyntheticCommandDataset.medium().len() == 1000
    m = audio.SyntheticMusicDataset.medium()
    assert (m.len(), m.sample_rate(), m.num_genres(), m.get(1)[0].numel()) == (500, 22050, 10, 44100) and audio.SyntheticMusicDataset.small().num_genres() == 5
    sp = audio.SyntheticSpeakerDataset.medium()
    assert (sp.len(), sp.num_speakers(), sp.sample_rate()) == (500, 20, 16000) and audio.SyntheticSpeakerDataset.small().num_speakers() == 5
    assert audio.SyntheticSpeakerDataset(10, 1).num_speakers() == 2                       # at least two speakers
    t = audio.TrimSilence.default_threshold()
    assert t.threshold_db == -60.0 and t.thr == pytest.approx(1e-3)
    w = torch.cat([torch.zeros(100), torch.ones(50), torch.zeros(30)])
    assert t(w).numel() == 50 and audio.TrimSilence.new(-20.0).threshold_db == -20.0
