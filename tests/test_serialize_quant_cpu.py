"""Checkpoint formats (bincode StateDict with golden bytes, checkpoints, SafeTensors, JSON, key
conversion), block quantisation against hand-computed blocks, GGUF round trips, ONNX export/import."""
import struct

import numpy as np
import pytest
import torch

from axonml_b200 import nn, onnx, optim, quant, serialize
from axonml_b200.quant import QuantType
from axonml_b200.serialize import codec
from axonml_b200.serialize.state_dict import StateDict


def test_state_dict_bincode_golden_bytes():
    """bincode 1.x layout of StateDict{entries: HashMap<String, {data:{shape:Vec<usize>,
    values:Vec<f32>}, requires_grad:bool, metadata:HashMap}>, metadata: HashMap}."""
    sd = StateDict.from_tensors({"w": torch.tensor([[1.0, 2.0]])})
    raw = codec.encode_state_dict(sd)
    golden = (struct.pack("<Q", 1) + struct.pack("<Q", 1) + b"w"            # one entry, key "w"
              + struct.pack("<Q", 2) + struct.pack("<QQ", 1, 2)             # shape [1, 2]
              + struct.pack("<Q", 2) + struct.pack("<ff", 1.0, 2.0)         # values
              + b"\x01" + struct.pack("<Q", 0)                              # requires_grad, entry metadata
              + struct.pack("<Q", 0))                                       # dict metadata
    assert raw == golden
    back, _ = codec.decode_state_dict(raw) if isinstance(codec.decode_state_dict(raw), tuple) else (codec.decode_state_dict(raw), None)
    assert torch.equal(back.to_tensors()["w"], torch.tensor([[1.0, 2.0]]))


def test_formats_round_trip(tmp_path):
    torch.manual_seed(0)
    m = nn.Sequential().add(nn.Linear(4, 3)).add(nn.ReLU()).add(nn.Linear(3, 2))
    sd = StateDict.from_module(m)
    for name, fmt in (("a.axonml", None), ("a.json", None), ("a.safetensors", None)):
        p = str(tmp_path / name)
        serialize.save_state_dict(sd, p)
        assert serialize.detect_format(p).value in name
        back = serialize.load_state_dict(p).to_tensors()
        for k, v in sd.to_tensors().items():
            assert torch.allclose(back[k], v), (name, k)
    # SafeTensors header is 8-byte LE length + JSON
    raw = open(str(tmp_path / "a.safetensors"), "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    assert raw[8:8 + n].lstrip().startswith(b"{")
    m2 = nn.Sequential().add(nn.Linear(4, 3)).add(nn.ReLU()).add(nn.Linear(3, 2))
    serialize.save_model(m, str(tmp_path / "m.axonml"))
    serialize.load_model(m2, str(tmp_path / "m.axonml"))
    x = torch.randn(2, 4)
    assert torch.allclose(m(x), m2(x))


def test_checkpoint_resume_bit_exact(tmp_path):
    torch.manual_seed(1)
    model = nn.Linear(3, 2)
    opt = optim.Adam(list(model.parameters()), 0.01)
    for _ in range(3):
        opt.zero_grad(); model(torch.ones(1, 3)).sum().backward(); opt.step()
    ts = serialize.TrainingState()
    ts.epoch, ts.global_step = 2, 30
    ck = (serialize.Checkpoint.builder().model_state(StateDict.from_module(model))
          .optimizer_state(serialize.optimizer_to_state_dict(opt)).training_state(ts).config("lr", 0.01).build())
    p = str(tmp_path / "c.axonml")
    serialize.save_checkpoint(ck, p)
    back = serialize.load_checkpoint(p)
    assert back.epoch() == 2 and back.global_step() == 30 and back.config["lr"] == "0.01"
    model2 = nn.Linear(3, 2)
    opt2 = optim.Adam(list(model2.parameters()), 0.01)
    back.model_state.load_into(model2)
    serialize.optimizer_from_state_dict(opt2, back.optimizer_state)
    for mm, oo in ((model, opt), (model2, opt2)):
        oo.zero_grad(); mm(torch.ones(1, 3)).sum().backward(); oo.step()
    assert torch.equal(model.weight, model2.weight)


def test_pytorch_key_conversion():
    assert serialize.convert_from_pytorch_key("module.layer.weight") == "layer.weight"
    sd = serialize.from_pytorch_state_dict({"module.fc.weight": torch.ones(2, 2)})
    assert list(sd.keys()) == ["fc.weight"]


def test_q8_0_and_q4_0_blocks_by_hand():
    x = torch.linspace(-1.0, 1.0, 32)
    q = quant.quantize_tensor(x, QuantType.Q8_0)
    raw = q.data.numpy().tobytes()
    assert len(raw) == 34
    d = np.frombuffer(raw[:2], dtype=np.float16)[0]
    assert abs(float(d) - 1.0 / 127.0) < 1e-4
    qs = np.frombuffer(raw[2:], dtype=np.int8)
    assert qs[0] == -127 and qs[-1] == 127
    deq = quant.dequantize_tensor(q)
    assert (deq - x).abs().max() < 1.0 / 127.0
    q4 = quant.quantize_tensor(x, QuantType.Q4_0)
    assert q4.data.numel() == 18
    assert (quant.dequantize_tensor(q4) - x).abs().max() < 0.2


@pytest.mark.parametrize("qt,tol", [(QuantType.Q8_0, 0.01), (QuantType.Q4_0, 0.15), (QuantType.Q4_1, 0.1),
                                    (QuantType.Q5_0, 0.08), (QuantType.Q5_1, 0.05), (QuantType.Q4_K, 0.12)])
def test_quantise_round_trip_error(qt, tol):
    torch.manual_seed(0)
    w = torch.randn(8, 512)
    q = quant.quantize_tensor(w, qt)
    assert q.size_bytes() == w.numel() // qt.block_size() * qt.bytes_per_block()
    d = quant.dequantize_tensor(q).view_as(w)
    assert quant.compute_quantization_error(w, d) < tol * float(w.std()) * 2


def test_gguf_round_trip(tmp_path):
    torch.manual_seed(0)
    w = torch.randn(4, 256)
    b = torch.randn(7)
    p = str(tmp_path / "t.gguf")
    quant.write_gguf(p, {"w": quant.quantize_tensor(w, QuantType.Q4_K), "w8": w, "b": b},
                     {"general.name": "t", "llama.block_count": 2}, quant={"w8": QuantType.Q8_0})
    raw = open(p, "rb").read()
    assert raw[:4] == b"GGUF" and struct.unpack("<I", raw[4:8])[0] == 3
    g = quant.read_gguf(p)
    assert g.metadata["general.name"] == "t" and g.metadata["llama.block_count"] == 2
    assert sorted(g.tensor_names()) == ["b", "w", "w8"]
    assert torch.equal(g.tensor("b"), b)
    qw = g.quantized("w")
    assert qw.quant_type is QuantType.Q4_K and list(qw.shape) == [4, 256]
    assert torch.equal(qw.data, quant.quantize_tensor(w, QuantType.Q4_K).data)
    assert (g.tensor("w8") - w).abs().max() < 0.05


def test_calibration():
    c = quant.calibrate(torch.tensor([-2.0, 0.0, 4.0]))
    assert c.min == -2.0 and c.max == 4.0 and abs(c.symmetric_scale(QuantType.Q8_0) - 4.0 / 127.0) < 1e-6


def test_onnx_export_import_matches_module(tmp_path):
    torch.manual_seed(0)
    m = nn.Sequential().add(nn.Linear(6, 5)).add(nn.ReLU()).add(nn.Linear(5, 3))
    ex = onnx.export_module(m, [1, 6], "mlp")
    p = str(tmp_path / "m.onnx")
    onnx.export_onnx(ex, p)
    model = onnx.import_onnx(p)
    x = torch.randn(4, 6)
    out = model.forward({"input": x})
    y = list(out.values())[0] if isinstance(out, dict) else out
    assert torch.allclose(y, m(x), atol=1e-5)
    assert model.num_parameters() == 6 * 5 + 5 + 5 * 3 + 3


def test_onnx_messages_round_trip_an_exported_model(tmp_path):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(6, 5), nn.ReLU(), nn.Linear(5, 3))
    data = onnx.export_module(m, [1, 6], "mlp").to_bytes()
    mp = onnx.ModelProto.from_bytes(data)
    assert mp.opset_version() == 17 == onnx.SUPPORTED_OPSET_VERSION and mp.producer_name == "axonml_b200" and mp.graph.name == "mlp"
    g = mp.graph
    assert [n.op_type for n in g.node] == ["Gemm", "Relu", "Gemm", "Identity"] and g.node[0].get_int("transB") == 1 and g.node[0].get_float("alpha", 1.0) == 1.0
    assert [v.name for v in g.graph_inputs()] == ["input"] and g.graph_inputs()[0].shape() == [None, 6] and len(g.initializer) == 4
    w0 = g.get_initializer(g.node[0].input[1])
    assert w0 is not None and w0.dims == [5, 6] and w0.data_type == onnx.TensorDataType.Float and w0.numel() == 30
    assert torch.equal(w0.to_tensor(), m[0].weight.detach()) and w0.get_float_data() == m[0].weight.detach().reshape(-1).tolist()
    assert set(g.initializer_map()) == {t.name for t in g.initializer} and g.get_initializer("nope") is None
    # the object model writes the same model back: the interpreter gives the same answer from the re-encoded bytes
    again = onnx.ModelProto.from_bytes(mp.to_bytes())
    assert again == mp
    x = torch.randn(1, 6)
    y1 = onnx.import_onnx_bytes(data).forward({"input": x})
    y2 = onnx.import_onnx_bytes(mp.to_bytes()).forward({"input": x})
    assert torch.equal(list(y1.values())[0], list(y2.values())[0]) and torch.allclose(list(y1.values())[0], m(x), atol=1e-5)
    # edit and save: rename the graph, add metadata, change an attribute
    mp.graph.name = "edited"
    mp.metadata_props.append(onnx.StringStringEntry("author", "test"))
    mp.graph.node[1] = onnx.NodeProto(list(g.node[0].output), list(g.node[1].output), "act", "LeakyRelu", attribute=[onnx.AttributeProto.float("alpha", 0.5)])
    p = tmp_path / "edited.onnx"
    mp.save(p)
    back = onnx.ModelProto.load(p)
    assert back.graph.name == "edited" and back.metadata() == {"author": "test"} and back.graph.node[1].get_float("alpha") == 0.5
    y3 = list(onnx.import_onnx(str(p)).forward({"input": x}).values())[0]
    want = torch.nn.functional.leaky_relu(m[0](x), 0.5) @ m[2].weight.t() + m[2].bias
    assert torch.allclose(y3, want, atol=1e-5)


def test_onnx_message_types_and_accessors():
    T = onnx.TensorDataType
    assert T.Float.size_bytes() == 4 and T.Bfloat16.size_bytes() == 2 and T.String.size_bytes() == 0 and T.from_i32(7) is T.Int64 and T.from_i32(99) is None
    assert T.Float16.torch_dtype() is torch.float16 and T.Int64.numpy_dtype() == "<i8"
    d = onnx.Dimension.fixed(3)
    assert d.value() == 3 and onnx.Dimension.dynamic("batch").value() is None and onnx.Dimension.from_bytes(d.to_bytes()) == d
    assert onnx.Dimension.from_bytes(onnx.Dimension.dynamic("batch").to_bytes()).dim_param == "batch"
    sh = onnx.TensorShape.from_dims([-1, 3, 224, 224])
    assert sh.to_vec() == [None, 3, 224, 224] and onnx.TensorShape.from_bytes(sh.to_bytes()) == sh
    vi = onnx.ValueInfo.tensor("x", ["N", 4], T.Int64)
    got = onnx.ValueInfo.from_bytes(vi.to_bytes())
    assert got == vi and got.shape() == [None, 4] and got.type.tensor_type.elem_type == T.Int64
    t = onnx.TensorProto.float("w", [2, 2], [1, 2, 3, 4])
    assert onnx.TensorProto.from_bytes(t.to_bytes()) == t and t.to_tensor().tolist() == [[1.0, 2.0], [3.0, 4.0]] and t.get_int64_data() == [1, 2, 3, 4]
    for src in (torch.arange(6, dtype=torch.int64).view(2, 3), torch.tensor([True, False]), torch.randn(3).half(), torch.randn(2, 2).double(),
                torch.tensor([1, -2], dtype=torch.int8)):
        tp = onnx.TensorProto.from_tensor("t", src)
        rt = onnx.TensorProto.from_bytes(tp.to_bytes())
        assert rt == tp and torch.equal(rt.to_tensor(), src) and rt.numel() == src.numel()
    assert onnx.TensorProto.from_tensor("b", torch.ones(2, dtype=torch.bfloat16)).data_type == T.Float          # stored widened
    ints = onnx.TensorProto("i", [3], int(T.Int64), int64_data=[5, -6, 7])
    assert onnx.TensorProto.from_bytes(ints.to_bytes()).to_tensor().tolist() == [5, -6, 7]
    halves = onnx.TensorProto("h", [2], int(T.Float16), int32_data=[0x3C00, 0xC000])               # fp16 bit patterns of 1.0 and -2.0
    assert halves.to_tensor().tolist() == [1.0, -2.0]
    with pytest.raises(ValueError):
        onnx.TensorProto("s", [1], int(T.String)).to_numpy()
    A = onnx.AttributeProto
    attrs = [A.int("axis", -1), A.float("alpha", 0.25), A.string("mode", "tanh"), A.make_ints("perm", [1, 0, 2]), A.make_floats("scales", [0.5, 2.0]),
             A.tensor("value", t)]
    node = onnx.NodeProto(["a", "b"], ["c"], "n0", "Custom", "my.domain", attrs, "doc")
    back = onnx.NodeProto.from_bytes(node.to_bytes())
    assert back == node and back.get_int("axis") == -1 and back.get_float("alpha") == 0.25 and back.get_ints("perm") == [1, 0, 2]
    assert back.get_string("mode") == "tanh" and back.get_attribute("nope") is None and back.get_int("nope", 7) == 7
    vals = back.attrs()
    assert vals["scales"] == [0.5, 2.0] and vals["mode"] == "tanh" and torch.equal(vals["value"], t.to_tensor()) and A.int("k", 1).type == onnx.AttributeType.Int
    mp = onnx.ModelProto(opset_import=[onnx.OperatorSetIdProto("ai.onnx.ml", 3), onnx.OperatorSetIdProto(None, 13)], model_version=2)
    assert mp.opset_version() == 13 and onnx.ModelProto.from_bytes(mp.to_bytes()) == mp and onnx.ModelProto().opset_version() == 17
    assert mp.ir_version == onnx.ONNX_IR_VERSION == 8


def test_onnx_operator_objects():
    mk = lambda op, ins, outs=("y",), **a: onnx.NodeProto(list(ins), list(outs), None, op, attribute=[
        onnx.AttributeProto.float(k, v) if isinstance(v, float) else onnx.AttributeProto.make_ints(k, v) if isinstance(v, list) else onnx.AttributeProto.int(k, v)
        for k, v in a.items()])
    x = torch.tensor([[-1.0, 2.0], [3.0, -4.0]])
    relu = onnx.create_operator(mk("Relu", ["x"]))
    assert isinstance(relu, onnx.ReluOp) and relu.name() == "Relu" and relu.execute([x])[0].tolist() == [[0.0, 2.0], [3.0, 0.0]]
    leaky = onnx.create_operator(mk("LeakyRelu", ["x"], alpha=0.5))
    assert leaky.attrs == {"alpha": 0.5} and leaky([x])[0].tolist() == [[-0.5, 2.0], [3.0, -2.0]] and repr(leaky) == "LeakyReluOp(alpha=0.5)"
    w, b = torch.randn(3, 2), torch.randn(3)
    gemm = onnx.create_operator(mk("Gemm", ["x", "w", "b"], transB=1, alpha=2.0))
    assert torch.allclose(gemm.execute([x, w, b])[0], 2.0 * x @ w.t() + b) and torch.allclose(gemm.execute([x, w])[0], 2.0 * x @ w.t())
    assert onnx.create_operator(mk("Transpose", ["x"], perm=[1, 0])).execute([x])[0].tolist() == x.t().tolist()
    assert onnx.create_operator(mk("ReduceSum", ["x"], axes=[1], keepdims=0)).execute([x])[0].tolist() == [1.0, -1.0]
    assert onnx.create_operator(mk("Concat", ["a", "b", "c"], axis=0)).execute([x, x, x])[0].shape == (6, 2)
    assert onnx.create_operator(mk("Clip", ["x", "lo", "hi"])).execute([x, torch.tensor(-2.0), torch.tensor(2.5)])[0].tolist() == [[-1.0, 2.0], [2.5, -2.0]]
    assert onnx.create_operator(mk("Shape", ["x"])).execute([x])[0].tolist() == [2, 2]
    img, k = torch.randn(1, 2, 5, 5), torch.randn(3, 2, 3, 3)
    conv = onnx.create_operator(mk("Conv", ["x", "w"], pads=[1, 1, 1, 1], strides=[2, 2]))
    assert torch.allclose(conv.execute([img, k])[0], torch.nn.functional.conv2d(img, k, None, 2, 1)) and isinstance(conv, onnx.ConvOp)
    from_interp = onnx.create_operator(onnx.CompiledOp("Softmax", ["x"], ["y"], {"axis": 0}))
    assert torch.allclose(from_interp.execute([x])[0], torch.softmax(x, 0))
    with pytest.raises(onnx.UnsupportedOperator, match="Unsupported operator: Einsum") as e:
        onnx.create_operator(mk("Einsum", ["x"]))
    assert isinstance(e.value, onnx.OnnxError) and e.value.op_type == "Einsum"
    with pytest.raises(onnx.OnnxError, match="Add takes 2 inputs, got 1"):
        onnx.AddOp().execute([x])
    with pytest.raises(onnx.OnnxError, match="required input is missing"):
        onnx.AddOp().execute([x, None])
    with pytest.raises(onnx.OnnxError, match="Gemm takes 2 to 3 inputs"):
        onnx.GemmOp().execute([x])
    assert set(onnx.OPERATOR_CLASSES) == set(onnx.SUPPORTED_OPS) and onnx.OPERATOR_CLASSES["AveragePool"] is onnx.AvgPoolOp
    assert all(issubclass(c, onnx.OnnxOperator) for c in onnx.OPERATOR_CLASSES.values()) and onnx.BatchNormOp.ARITY == (5, 5)
