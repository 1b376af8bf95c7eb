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
