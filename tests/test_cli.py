"""Command line: project file round trip, train -> resume -> eval -> predict, convert, inspect,
quantise (real GGUF and the reference's fake-quant), ONNX export, hub, report."""
import json
import os

import pytest
import torch

from axonml_b200.cli import ProjectConfig, main


def test_project_config_round_trip(tmp_path):
    cfg = ProjectConfig()
    cfg.training.epochs = 3
    cfg.training.optimizer.name = "sgd"
    cfg.model.architecture = "lenet"
    cfg.distributed.tp = 8
    p = tmp_path / "axonml.toml"
    cfg.save(str(p))
    back = ProjectConfig.load(str(p))
    assert back == cfg
    assert back.validate() == []
    back.training.epochs = 0
    back.precision.dtype = "fp8"
    assert len(back.validate()) == 2


def test_train_resume_eval_predict_and_tools(tmp_path, capsys, monkeypatch):
    monkeypatch.chdir(tmp_path)
    main(["new", "proj"])
    assert os.path.exists("proj/axonml.toml")
    out = str(tmp_path / "out")
    common = ["--model", "mlp", "--data", "synthetic-mnist", "--device", "cpu", "--output", out]
    main(["train", *common, "--epochs", "2", "--batch-size", "64", "--lr", "0.003", "--optimizer", "adam"])
    ck2 = os.path.join(out, "checkpoint_epoch_2.axonml")
    assert os.path.exists(ck2)
    main(["resume", *common, "--epochs", "3", "--batch-size", "64", "--lr", "0.003", "--optimizer", "adam"])
    ck3 = os.path.join(out, "checkpoint_epoch_3.axonml")
    assert os.path.exists(ck3)
    capsys.readouterr()
    main(["eval", ck3, *common])
    acc = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["accuracy"]
    assert acc > 0.5          # the synthetic task is learnable in three epochs
    main(["predict", ck3, *common, "--index", "3"])
    pred = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert set(pred) == {"index", "label", "predicted", "confidence"}
    main(["inspect", ck3])
    assert "parameters" in capsys.readouterr().out
    st = str(tmp_path / "m.safetensors")
    main(["convert", ck3, st])
    back = str(tmp_path / "m2.axonml")
    main(["convert", st, back])
    from axonml_b200.serialize import load_state_dict
    b = load_state_dict(back)
    assert len(list(b.keys())) == 6
    gg = str(tmp_path / "m.gguf")
    main(["quant", back, gg, "--type", "q8_0"])
    main(["inspect", gg])
    assert "parameters" in capsys.readouterr().out
    fq = str(tmp_path / "fake.axonml")
    main(["quant", back, fq, "--type", "q4_0", "--fake"])
    assert len(list(load_state_dict(fq).keys())) == 6
    onx = str(tmp_path / "m.onnx")
    main(["export", onx, "--checkpoint", ck3, *common])
    assert os.path.getsize(onx) > 1000
    main(["report", out])
    txt = capsys.readouterr().out
    rows = json.loads(txt[txt.find("["):])
    assert [r["epoch"] for r in rows] == [1, 2, 3]
    main(["hub", "list"])
    assert "resnet" in capsys.readouterr().out.lower()
    main(["gpu"])
    assert "cuda_available" in capsys.readouterr().out


def _mlp_file(path, dims=(8, 16, 3), seed=0):
    from axonml_b200 import nn
    from axonml_b200.serialize import save_state_dict
    from axonml_b200.serialize.state_dict import StateDict
    torch.manual_seed(seed)
    layers = []
    for a, b in zip(dims, dims[1:]):
        layers += [nn.Linear(a, b), nn.ReLU()]
    net = nn.Sequential(*layers[:-1])
    save_state_dict(StateDict.from_module(net), str(path))
    return net.eval()


def _csv_data(path, net, n=60, seed=1):
    torch.manual_seed(seed)
    x = torch.randn(n, 8)
    with torch.no_grad():
        y = net(x).argmax(-1)
    flip = torch.arange(n) % 5 == 0                       # every fifth label is wrong on purpose
    y = torch.where(flip, (y + 1) % 3, y)
    with open(path, "w") as f:
        f.write(",".join(f"f{i}" for i in range(8)) + ",label\n")
        for r, l in zip(x.tolist(), y.tolist()):
            f.write(",".join(f"{v:.6f}" for v in r) + f",c{l}\n")
    return x, y


def test_model_file_commands_in_the_reference_syntax(tmp_path, capsys, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("AXONML_CONFIG_DIR", str(tmp_path / "cfg"))
    net = _mlp_file(tmp_path / "m.axonml")
    x, y = _csv_data(tmp_path / "d.csv", net)
    main(["eval", "m.axonml", "d.csv", "--metrics", "accuracy,loss,f1", "-b", "16"])
    ev = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ev["samples"] == 60 and ev["accuracy"] == pytest.approx(0.8) and ev["loss"] > 0 and 0 < ev["f1"] <= 1
    with pytest.raises(SystemExit, match="unknown metric"):
        main(["eval", "m.axonml", "d.csv", "-m", "bleu"])
    capsys.readouterr()
    # predict: comma-separated values, a JSON array of two samples with the top classes, a CSV file to a text file
    main(["predict", "m.axonml", ",".join(f"{v:.6f}" for v in x[0].tolist())])
    one = json.loads(capsys.readouterr().out)
    with torch.no_grad():
        want = net(x[:2]).softmax(-1)
    assert one["architecture"] == "sequential-mlp" and one["predictions"][0]["predicted"] == int(want[0].argmax())
    main(["predict", "m.axonml", json.dumps({"data": x[:2].tolist()}), "-t", "2"])
    two = json.loads(capsys.readouterr().out)["predictions"]
    assert len(two) == 2 and [t["class"] for t in two[1]["top_k"]] == want[1].topk(2).indices.tolist()
    assert two[1]["top_k"][0]["probability"] == pytest.approx(float(want[1].max()), abs=1e-5)
    (tmp_path / "in.csv").write_text("\n".join(",".join(f"{v:.6f}" for v in r) for r in x[:3].tolist()))
    main(["predict", "m.axonml", "in.csv", "-f", "text", "-o", "pred.txt"])
    assert open("pred.txt").read().count("sample ") == 3
    with pytest.raises(SystemExit, match="Cannot parse input"):
        main(["predict", "m.axonml", "nonsense"])
    capsys.readouterr()
    # report: html with every section, json, text; a history file feeds the loss curves
    with open("hist.jsonl", "w") as f:
        for e in range(1, 4):
            f.write(json.dumps({"epoch": e, "train_loss": 1.0 / e, "val_loss": 1.2 / e}) + "\n")
    main(["report", "m.axonml", "-d", "d.csv", "--history", "hist.jsonl", "-o", "rep.html"])
    page = open("rep.html").read()
    assert "Confusion matrix" in page and "Per-class metrics" in page and "<polyline" in page and "c0" in page
    assert "accuracy 0.8000" in capsys.readouterr().out
    main(["report", "m.axonml", "-d", "d.csv", "-f", "json", "-o", "rep.json", "--confusion-matrix", "false", "--class-names", "ants,bees,wasps"])
    rep = json.load(open("rep.json"))
    assert rep["metrics"]["accuracy"] == pytest.approx(0.8) and "confusion_matrix" not in rep["metrics"]
    assert [p["class_name"] for p in rep["metrics"]["per_class"]] == ["ants", "bees", "wasps"]
    assert sum(p["support"] for p in rep["metrics"]["per_class"]) == 60
    capsys.readouterr()
    main(["report", "m.axonml", "-d", "d.csv", "-f", "text"])
    txt = capsys.readouterr().out
    assert "Macro F1" in txt and "rows: true class" in txt
    with pytest.raises(SystemExit, match="needs --data"):
        main(["report", "m.axonml"])
    # inspect
    main(["inspect", "m.axonml", "-f", "json", "-d"])
    ins = json.loads(capsys.readouterr().out)
    assert ins["parameters"] == 8 * 16 + 16 + 16 * 3 + 3 and len(ins["entries"]) == 4 and ins["format"] == "axonml"
    main(["inspect", "m.axonml", "--show-params", "2", "-d"])
    out = capsys.readouterr().out
    assert "layers:" in out and "0.weight: [" in out and ", ...]" in out
    # export / convert
    main(["export", "m.axonml", "m.onnx"])
    from axonml_b200 import onnx
    got = list(onnx.import_onnx("m.onnx").forward({"input": x[:4]}).values())[0]
    with torch.no_grad():
        assert torch.allclose(got, net(x[:4]), atol=1e-5)
    main(["export", "m.axonml", "m.st", "-f", "safetensors", "--quantize", "--precision", "bf16"])
    from axonml_b200.serialize import load_state_dict
    from axonml_b200.serialize.codec import safetensors_loads
    stored, meta = safetensors_loads(open("m.st", "rb").read())
    assert all(v.dtype == torch.bfloat16 for v in stored.values()) and meta["architecture"] == "sequential-mlp"
    assert torch.equal(load_state_dict("m.st").to_tensors()["0.bias"], net[0].bias.detach().bfloat16().float())
    main(["export", "m.axonml", "m.gguf", "-f", "gguf", "--quantize", "--precision", "q8_0"])
    capsys.readouterr()
    main(["quant", "info", "m.gguf"])
    assert json.loads(capsys.readouterr().out)["tensors"] == 4
    main(["convert", "m.axonml", "m.pt"])
    raw = torch.load("m.pt", weights_only=True)
    assert set(raw) == {"0.weight", "0.bias", "2.weight", "2.bias"}
    main(["convert", "m.pt", "back.safetensors", "--from", "pytorch"])
    assert torch.equal(load_state_dict("back.safetensors").to_tensors()["2.weight"], raw["2.weight"])
    main(["convert", "m.axonml", "c.onnx", "--to", "onnx"])
    assert os.path.getsize("c.onnx") > 500
    with pytest.raises(SystemExit, match="unknown export format"):
        main(["export", "m.axonml", "m.xyz", "-f", "xyz"])


def test_quant_bench_gpu_hub_new_init_in_the_reference_syntax(tmp_path, capsys, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("AXONML_CONFIG_DIR", str(tmp_path / "cfg"))
    monkeypatch.setenv("AXONML_HUB_CACHE", str(tmp_path / "hubcache"))
    monkeypatch.setenv("AXONML_HUB_ENDPOINT", "http://127.0.0.1:9")
    _mlp_file(tmp_path / "big.axonml", dims=(64, 128, 64))
    _mlp_file(tmp_path / "small.axonml", dims=(64, 32, 64))
    main(["quant", "list"])
    assert "q4_k" in capsys.readouterr().out
    main(["quant", "convert", "big.axonml", "-t", "q4_0", "-o", "big.gguf"])
    assert "quantised 2 tensors to Q4_0" in capsys.readouterr().out
    with pytest.raises(SystemExit, match="exists"):
        main(["quant", "convert", "big.axonml", "-t", "q4_0", "-o", "big.gguf"])
    main(["quant", "convert", "big.axonml", "-t", "q8_0", "-o", "big.gguf", "--overwrite"])
    capsys.readouterr()
    main(["quant", "info", "big.gguf", "-d"])
    info = json.loads(capsys.readouterr().out)
    assert info["by_type"]["q8_0"]["tensors"] == 2 and info["parameters"] == 64 * 128 * 2 + 128 + 64 and len(info["entries"]) == 4
    assert 8.0 < info["bits_per_parameter"] < 12.0
    main(["quant", "benchmark", "big.axonml", "-i", "2", "-t", "q8_0,q4_0"])
    rows = json.loads(capsys.readouterr().out)["results"]
    assert [r["type"] for r in rows] == ["q8_0", "q4_0"] and rows[0]["mean_rmse"] < rows[1]["mean_rmse"]
    assert rows[0]["compression_ratio"] == pytest.approx(32 / 8.5, rel=1e-3) and rows[1]["compression_ratio"] == pytest.approx(32 / 4.5, rel=1e-3)
    with pytest.raises(SystemExit, match="unknown quantisation type"):
        main(["quant", "convert", "big.axonml", "-t", "q9_9", "-o", "x.gguf"])
    main(["bench", "model", "big.axonml", "-i", "5", "-w", "1", "-b", "4", "--device", "cpu"])
    b = json.loads(capsys.readouterr().out)
    assert b["batch_size"] == 4 and b["iterations"] == 5 and b["min_ms"] <= b["p50_ms"] <= b["max_ms"] and b["throughput_per_s"] > 0
    main(["bench", "inference", "big.axonml", "-b", "1,8", "-i", "3", "--device", "cpu", "-o", "inf.json"])
    assert [r["batch_size"] for r in json.load(open("inf.json"))["results"]] == [1, 8]
    capsys.readouterr()
    main(["bench", "compare", "big.axonml,small.axonml", "-i", "3", "--device", "cpu"])
    cmp_ = json.loads(capsys.readouterr().out)
    assert {r["model"] for r in cmp_["results"]} == {"big.axonml", "small.axonml"} and min(r["relative"] for r in cmp_["results"]) == 1.0
    with pytest.raises(SystemExit, match="needs a model file"):
        main(["bench", "compare"])
    main(["gpu", "status"])
    st = json.loads(capsys.readouterr().out)
    assert st["selected"] is None and st["device_count"] == (torch.cuda.device_count() if torch.cuda.is_available() else 0)
    main(["gpu", "select", "cpu", "-p"])
    assert json.loads(capsys.readouterr().out) == {"selected": "cpu", "persistent": True}
    main(["gpu", "status"])
    assert json.loads(capsys.readouterr().out)["selected"] == "cpu"
    with pytest.raises(SystemExit, match="no such GPU"):
        main(["gpu", "select", "63"])
    main(["gpu", "memory"]); main(["gpu", "list"]); main(["gpu", "info"])
    assert "cuda_available" in capsys.readouterr().out
    main(["hub", "list"])
    out = capsys.readouterr().out
    assert "pretrained weights:" in out and "resnet18" in out and "tinyllama-1.1b" in out
    main(["hub", "info", "resnet18"])
    inf = json.loads(capsys.readouterr().out)
    assert inf["pretrained"]["accuracy"] == 69.76 and inf["weights_cached"] is False and inf["architecture"] == "ResNet"
    main(["hub", "info", "phi-2"])
    assert json.loads(capsys.readouterr().out)["pretrained"]["hidden_size"] == 2560
    with pytest.raises(SystemExit, match="Network error"):
        main(["hub", "download", "bert-tiny"])
    with pytest.raises(SystemExit, match="no pretrained weights"):
        main(["hub", "download", "no-such-model"])
    os.makedirs(tmp_path / "hubcache" / "llm", exist_ok=True)
    (tmp_path / "hubcache" / "llm" / "bert-tiny.safetensors").write_bytes(b"x" * 10)
    main(["hub", "download", "bert-tiny"])                                # already cached: no network needed
    assert capsys.readouterr().out.strip().endswith("bert-tiny.safetensors")
    main(["hub", "cached"])
    assert "bert-tiny.safetensors" in capsys.readouterr().out
    main(["hub", "clear", "bert-tiny"])
    assert "removed 1" in capsys.readouterr().out and not os.path.exists(tmp_path / "hubcache" / "llm" / "bert-tiny.safetensors")
    main(["new", "proj", "-t", "lenet", "--no-git", "-p", "work"])
    cfg = ProjectConfig.load("work/proj/axonml.toml")
    assert cfg.model.architecture == "lenet" and cfg.project.name == "proj" and not os.path.exists("work/proj/.git")
    with pytest.raises(SystemExit, match="unknown template"):
        main(["new", "p2", "-t", "gan"])
    os.makedirs("here")
    monkeypatch.chdir(tmp_path / "here")
    main(["init", "-n", "named"])
    assert ProjectConfig.load("axonml.toml").project.name == "named"
    with pytest.raises(SystemExit):
        main(["init"])
    main(["init", "-f"])
    assert ProjectConfig.load("axonml.toml").project.name == "here"


def test_train_takes_a_data_path_and_resume_a_positional_checkpoint(tmp_path, capsys, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("AXONML_CONFIG_DIR", str(tmp_path / "cfg"))
    main(["dataset", "download", "mnist", "--output", "mnist"])
    main(["train", "-m", "mlp", "-d", "mnist", "-e", "1", "-b", "64", "-l", "0.003", "-o", "out", "--device", "cpu", "--workers", "0"])
    ck = "out/checkpoint_epoch_1.axonml"
    assert os.path.exists(ck)
    main(["resume", ck, "-m", "mlp", "-d", "mnist", "-e", "2", "-o", "out", "--device", "cpu"])
    assert os.path.exists("out/checkpoint_epoch_2.axonml")
    capsys.readouterr()
    main(["eval", "out/checkpoint_epoch_2.axonml", "mnist", "--format", "mnist"])
    ev = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ev["samples"] > 100 and 0.0 <= ev["accuracy"] <= 1.0
    main(["report", "out/checkpoint_epoch_2.axonml", "-d", "mnist", "-f", "text"])
    txt = capsys.readouterr().out
    assert "epoch  train_loss" in txt                                  # the run's own training_log.jsonl is picked up
