"""Unit tests of serialisation and ONNX on the CPU, one behaviour per test (the topics of the
reference's in-module tests under crates/axonml-serialize and crates/axonml-onnx)."""
import pytest
import torch

from axonml_b200 import nn, onnx as OX, serialize as S
from axonml_b200.serialize import Format, StateDict, TensorData, TrainingState


# ------------------------------------------------------------------------------------ state dict
def test_tensor_data_round_trip():
    t = torch.arange(6.0).reshape(2, 3)
    d = TensorData.from_tensor(t)
    assert d.shape == [2, 3] and d.numel() == 6 and d.to_tensor().equal(t)


def test_state_dict_insert_get_remove():
    sd = StateDict.new()
    assert sd.is_empty()
    sd.insert("fc.weight", TensorData.from_tensor(torch.ones(2, 3)))
    sd.insert("fc.bias", TensorData.from_tensor(torch.zeros(2)))
    assert sd.len() == 2 and sd.contains("fc.bias") and not sd.contains("missing") and sd.get("missing") is None
    assert list(sd.keys()) == ["fc.weight", "fc.bias"] and sd.total_params() == 8 and sd.size_bytes() == 32
    assert sd.get("fc.weight").data.to_tensor().sum().item() == 6
    sd.remove("fc.bias")
    assert sd.len() == 1


def test_state_dict_prefix_operations_and_merge():
    sd = StateDict.from_tensors({"enc.w": torch.ones(2), "enc.b": torch.ones(1), "dec.w": torch.ones(3)})
    enc = sd.filter_prefix("enc.")
    assert sorted(enc.keys()) == ["enc.b", "enc.w"]
    assert sorted(enc.strip_prefix("enc.").keys()) == ["b", "w"]
    assert sorted(enc.strip_prefix("enc.").add_prefix("x.").keys()) == ["x.b", "x.w"]
    other = StateDict.from_tensors({"head.w": torch.ones(4)})
    sd.merge(other)
    assert sd.len() == 4 and sd.contains("head.w")
    text = sd.summary()
    assert "4" in text and "10" in text                                    # entries and parameters


def test_state_dict_from_module_and_back():
    a, b = nn.Linear(3, 2), nn.Linear(3, 2)
    sd = StateDict.from_module(a)
    assert sorted(sd.keys()) == ["bias", "weight"]
    sd.load_into(b)
    assert torch.equal(a.weight, b.weight) and torch.equal(a.bias, b.bias)
    sd.set_metadata("note", "hello")
    assert sd.get_metadata("note") == "hello" and sd.get_metadata("none") is None


# ---------------------------------------------------------------------------------------- formats
def test_format_detection_from_extension_and_properties():
    assert S.detect_format("m.axonml") is Format.Axonml and S.detect_format("m.bin") is Format.Axonml
    assert S.detect_format("m.json") is Format.Json and S.detect_format("m.safetensors") is Format.SafeTensors
    assert S.detect_format("m.gguf") is Format.Gguf and S.detect_format("m.unknown") is Format.Axonml
    assert Format.Json.extension() == "json" and not Format.Json.is_binary() and Format.Axonml.is_binary()
    assert Format.SafeTensors.supports_streaming() and not Format.Json.supports_streaming() and len(Format.all()) == 4
    assert Format.Gguf.name_str() == "GGUF"


def test_format_detection_from_bytes():
    assert S.detect_format_from_bytes(b'{"a": 1}') is Format.Json
    assert S.detect_format_from_bytes(b"GGUF\x03\x00\x00\x00") is Format.Gguf
    assert S.detect_format_from_bytes(b"") is None


@pytest.mark.parametrize("ext", ["axonml", "json", "safetensors"])
def test_state_dict_round_trip_through_every_container(tmp_path, ext):
    sd = StateDict.from_tensors({"w": torch.randn(3, 4), "b": torch.arange(3.0)})
    path = str(tmp_path / f"m.{ext}")
    S.save_state_dict(sd, path)
    back = S.load_state_dict(path).to_tensors()
    assert set(back) == {"w", "b"} and torch.allclose(back["w"], sd.to_tensors()["w"], atol=1e-6) and back["b"].tolist() == [0, 1, 2]


def test_save_and_load_model(tmp_path):
    a, b = nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2)), nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2))
    S.save_model(a, str(tmp_path / "m.safetensors"))
    S.load_model(b, str(tmp_path / "m.safetensors"))
    x = torch.randn(5, 4)
    assert torch.allclose(a(x), b(x))
    with pytest.raises(Exception):
        S.load_model(nn.Linear(4, 3), str(tmp_path / "m.safetensors"), strict=True)


# ------------------------------------------------------------------------------------ checkpoints
def test_training_state_records_losses_and_epochs():
    ts = TrainingState.new()
    assert ts.epoch == 0 and ts.global_step == 0 and ts.avg_loss(5) is None
    for v in (4.0, 2.0, 3.0):
        ts.record_loss(v)
        ts.next_step()
    assert ts.global_step == 3 and ts.step == 3 and ts.avg_loss(2) == 2.5 and ts.avg_loss(10) == 3.0
    ts.record_val_loss(1.5)
    ts.record_lr(0.01)
    ts.record_metric("acc", 0.9)
    ts.next_epoch()
    assert ts.epoch == 1 and ts.step == 0 and ts.val_loss_history == [1.5] and ts.lr_history == [0.01] and ts.custom_metrics["acc"] == [0.9]


def test_training_state_best_metric_in_both_directions():
    ts = TrainingState.new()
    assert ts.update_best("loss", 1.0, False) and not ts.update_best("loss", 1.2, False) and ts.update_best("loss", 0.8, False)
    assert ts.best_metric == 0.8 and ts.best_metric_name == "loss"
    acc = TrainingState.new()
    assert acc.update_best("acc", 0.5, True) and acc.update_best("acc", 0.7, True) and not acc.update_best("acc", 0.6, True)


def test_checkpoint_builder_and_binary_round_trip(tmp_path):
    model = nn.Linear(3, 2)
    ts = TrainingState.new()
    ts.record_loss(0.5)
    ck = (S.Checkpoint.builder().model_state(StateDict.from_module(model)).training_state(ts).epoch(3).global_step(120)
          .config("lr", "0.01").rng_state(b"\x01\x02").build())
    assert ck.epoch() == 3 and ck.global_step() == 120 and ck.config["lr"] == "0.01" and ck.axonml_version
    back = S.decode_checkpoint(S.encode_checkpoint(ck))
    assert back.epoch() == 3 and back.rng_state == b"\x01\x02" and back.training_state.loss_history == [0.5]
    assert torch.equal(back.model_state.to_tensors()["weight"], model.weight.detach())
    S.save_checkpoint(ck, str(tmp_path / "c.axonml"))
    assert S.load_checkpoint(str(tmp_path / "c.axonml")).global_step() == 120


def test_checkpoint_builder_defaults_to_empty_states():
    ck = S.Checkpoint.builder().epoch(1).build()
    assert ck.epoch() == 1 and ck.model_state.is_empty() and ck.optimizer_state.is_empty() and ck.rng_state is None


def test_optimizer_state_survives_a_checkpoint():
    from axonml_b200 import optim
    p = nn.Parameter.new(torch.ones(3))
    o = optim.Adam([p], lr=0.1)
    p.grad = torch.ones(3)
    o.step()
    sd = S.optimizer_to_state_dict(o)
    q = nn.Parameter.new(p.detach().clone())
    o2 = optim.Adam([q], lr=0.1)
    S.optimizer_from_state_dict(o2, sd)
    p.grad, q.grad = torch.ones(3), torch.ones(3)
    o.step(), o2.step()
    assert torch.allclose(p.detach(), q.detach())


# ------------------------------------------------------------------------------------ conversion
def test_pytorch_key_conversion_both_ways():
    assert S.from_pytorch_key("module.encoder.0.weight") == "encoder.0.weight"
    assert S.from_pytorch_key("layer.running_mean") == "layer.running_mean"
    assert S.to_pytorch_key("encoder.0.weight") == "encoder.0.weight"
    sd = StateDict.from_tensors({"module.fc.weight": torch.ones(2, 2)})
    assert list(S.convert_from_pytorch(sd).keys()) == ["fc.weight"]
    assert isinstance(S.pytorch_layer_mapping(), dict) and S.pytorch_layer_mapping()


def test_linear_weights_are_transposed_and_biases_left_alone():
    sd = StateDict.from_tensors({"fc.weight": torch.arange(6.0).reshape(2, 3), "fc.bias": torch.zeros(2), "conv.weight": torch.zeros(2, 3, 1, 1)})
    t = S.transpose_linear_weights(sd).to_tensors()
    assert t["fc.weight"].shape == (3, 2) and t["fc.weight"][1, 0].item() == 1.0 and t["fc.bias"].shape == (2,) and t["conv.weight"].shape == (2, 3, 1, 1)


def test_onnx_shapes_and_operator_names():
    assert S.to_onnx_shape([3, 4]) == [3, 4] and S.to_onnx_shape([3, 4], include_batch=True) == [-1, 3, 4]
    assert S.from_onnx_shape([-1, 3, 4]) == [1, 3, 4] and S.from_onnx_shape([-1, 8], default_dynamic=16) == [16, 8]
    T = S.OnnxOpType
    assert T.from_str("Relu") is T.Relu and T.Gemm.as_str() == "Gemm" and T.from_str("NoSuchOp") is T.Unknown
    for t in T:
        assert T.from_str(t.as_str()) is t


# ------------------------------------------------------------------------------------------ ONNX
def test_onnx_tensor_proto_and_data_types():
    D = OX.TensorDataType
    assert int(D.Float) == 1 and int(D.Int64) == 7 and int(D.Double) == 11 and int(D.Bfloat16) == 16
    t = OX.TensorProto.from_tensor("w", torch.arange(6.0).reshape(2, 3)) if hasattr(OX.TensorProto, "from_tensor") else None
    assert t.name == "w" and t.dims == [2, 3] and OX.TensorProto.from_bytes(t.to_bytes()).to_tensor().equal(torch.arange(6.0).reshape(2, 3))
    i = OX.TensorProto.from_tensor("idx", torch.tensor([1, 2, 3]))
    assert i.data_type == int(D.Int64) and OX.TensorProto.from_bytes(i.to_bytes()).to_tensor().tolist() == [1, 2, 3]


def test_onnx_attribute_constructors_and_node_accessors():
    a = OX.AttributeProto
    node = OX.NodeProto(["x"], ["y"], "pool", "MaxPool", None,
                        [a.make_ints("kernel_shape", [2, 2]), a.int("ceil_mode", 0), a.float("alpha", 0.5), a.string("auto_pad", "NOTSET")])
    back = OX.NodeProto.from_bytes(node.to_bytes())
    assert back.op_type == "MaxPool" and back.input == ["x"] and back.get_ints("kernel_shape") == [2, 2]
    assert back.get_int("ceil_mode") == 0 and back.get_float("alpha") == 0.5 and back.get_string("auto_pad") == "NOTSET"
    assert back.get_int("missing", 7) == 7 if back.get_int.__code__.co_argcount > 2 else back.get_attribute("missing") is None


def test_onnx_operator_objects_compute():
    x = torch.tensor([[-1.0, 2.0], [3.0, -4.0]])
    assert OX.ReluOp().execute([x])[0].tolist() == [[0, 2], [3, 0]]
    assert OX.AddOp().execute([x, torch.ones(2)])[0].tolist() == [[0, 3], [4, -3]]
    assert torch.allclose(OX.MatMulOp().execute([x, torch.eye(2)])[0], x)
    assert OX.ReluOp().name() == "Relu" and OX.ReluOp.OP_TYPE == "Relu"
    with pytest.raises(Exception):
        OX.AddOp().execute([x])
    op = OX.create_operator(OX.NodeProto(["a"], ["b"], None, "Sigmoid"))
    assert torch.allclose(op.execute([x])[0], torch.sigmoid(x))
    with pytest.raises(OX.UnsupportedOperator):
        OX.create_operator(OX.NodeProto(["a"], ["b"], None, "NoSuchOp"))


def test_onnx_pooling_operators():
    x = torch.arange(16.0).reshape(1, 1, 4, 4)
    mp = OX.MaxPoolOp(kernel_shape=[2, 2], strides=[2, 2]).execute([x])[0]
    assert mp.flatten().tolist() == [5, 7, 13, 15]
    padded = OX.MaxPoolOp(kernel_shape=[3, 3], strides=[1, 1], pads=[1, 1, 1, 1]).execute([x])[0]
    assert padded.shape == (1, 1, 4, 4) and padded[0, 0, 0, 0].item() == 5.0
    ap = OX.AvgPoolOp(kernel_shape=[2, 2], strides=[2, 2]).execute([x])[0]
    assert ap.flatten().tolist() == [2.5, 4.5, 10.5, 12.5]
    multi = OX.MaxPoolOp(kernel_shape=[2, 2], strides=[2, 2]).execute([torch.randn(3, 5, 8, 8)])[0]
    assert multi.shape == (3, 5, 4, 4)
    assert OX.GlobalAveragePoolOp().execute([x])[0].flatten().tolist() == [7.5]


def test_exporter_builds_a_loadable_model():
    ex = OX.OnnxExporter.new("tiny").with_producer("axonml", "test") if hasattr(OX.OnnxExporter, "with_producer") else OX.OnnxExporter("tiny")
    ex.add_input("x", [1, 3])
    ex.add_initializer("w", torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]))
    ex.add_node("MatMul", ["x", "w"], ["h"])
    ex.add_named_node("act", "Relu", ["h"], ["y"])
    ex.add_output("y", [1, 2])
    model = OX.import_onnx_bytes(ex.to_bytes())
    out = model.forward({"x": torch.tensor([[1.0, -2.0, 0.5]])})
    y = out["y"] if isinstance(out, dict) else out
    assert y.tolist() == [[1.5, 0.0]] and model.num_parameters() == 6
    assert [i.name for i in model.get_inputs()] == ["x"] and model.get_inputs()[0].shape == [1, 3]
    proto = ex.to_proto()
    assert proto.graph.name == "tiny" and [n.op_type for n in proto.graph.node] == ["MatMul", "Relu"]


def test_exported_module_matches_the_module(tmp_path):
    m = nn.Sequential(nn.Linear(4, 6), nn.ReLU(), nn.Linear(6, 2)).eval()
    path = str(tmp_path / "m.onnx")
    OX.export_onnx(OX.export_module(m, [1, 4]), path)
    loaded = OX.import_onnx(path)
    x = torch.randn(3, 4)
    out = loaded.forward({loaded.get_inputs()[0].name: x})
    y = next(iter(out.values())) if isinstance(out, dict) else out
    assert torch.allclose(y, m(x), atol=1e-5)
    sd = loaded.to_state_dict()
    assert sum(v.numel() for v in (sd.to_tensors() if hasattr(sd, "to_tensors") else sd).values()) == m.num_parameters()


def test_feedforward_export_helper():
    layers = [(torch.randn(5, 3), torch.randn(5)), (torch.randn(2, 5), torch.randn(2))]
    model = OX.import_onnx_bytes(OX.export_onnx_bytes(OX.export_feedforward("ff", layers, 3)))
    x = torch.randn(4, 3)
    out = model.forward({"input": x})
    y = next(iter(out.values())) if isinstance(out, dict) else out
    ref = torch.relu(x @ layers[0][0].t() + layers[0][1]) @ layers[1][0].t() + layers[1][1]
    assert torch.allclose(y, ref, atol=1e-5)


def test_model_proto_round_trip_and_metadata():
    ex = OX.OnnxExporter("meta")
    ex.add_input("x", [2])
    ex.add_node("Identity", ["x"], ["y"])
    ex.add_output("y", [2])
    proto = ex.to_proto()
    proto.metadata_props.append(OX.StringStringEntry("author", "tests"))
    back = OX.ModelProto.from_bytes(proto.to_bytes())
    assert back.ir_version == proto.ir_version and back.opset_import[0].version >= 13
    assert [(e.key, e.value) for e in back.metadata_props] == [("author", "tests")]
    assert back.graph.graph_inputs()[0].name == "x" if hasattr(back.graph, "graph_inputs") else back.graph.input[0].name == "x"


def test_importing_garbage_fails_cleanly():
    with pytest.raises(Exception):
        OX.import_onnx_bytes(b"\xff\xff\xff\xff not a model")
