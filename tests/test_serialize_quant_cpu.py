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
