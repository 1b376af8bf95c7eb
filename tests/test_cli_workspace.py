"""Workspace, service and integration commands of the CLI, the TUI renderer and the offline
Kaggle / W&B clients (CPU only)."""
import json
import os
import subprocess
import sys
import zipfile

import pytest
import torch

from axonml_b200.cli.main import main as cli


@pytest.fixture()
def ws(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("AXONML_HOME", str(tmp_path / "home"))
    monkeypatch.setenv("AXONML_CONFIG_DIR", str(tmp_path / "cfg"))
    monkeypatch.setenv("KAGGLE_CONFIG_DIR", str(tmp_path / "kaggle"))
    return tmp_path


def _model_file(path):
    from axonml_b200 import nn
    from axonml_b200.serialize import save_state_dict
    from axonml_b200.serialize.state_dict import StateDict
    torch.manual_seed(0)
    save_state_dict(StateDict.from_module(nn.Sequential(nn.Linear(784, 32), nn.ReLU(), nn.Linear(32, 10))), str(path))


def test_dataset_catalogue_download_analyze_load_and_compatibility(ws, capsys):
    cli(["dataset", "list", "--source", "builtin"])
    assert "cifar-100" in capsys.readouterr().out
    cli(["dataset", "download", "mnist", "--output", "datasets/mnist"])
    from axonml_b200.vision.datasets import MNIST
    ds = MNIST("datasets/mnist", train=True)                      # the real loader reads the stand-in
    assert ds.len() == 1792 and ds.get(0)[0].shape == (1, 28, 28)
    cli(["data", "analyze", "datasets/mnist", "--format", "json", "--output", "an.json", "--recommend"])
    an = json.load(open("an.json"))
    assert an["dataset_type"] == "idx" and an["num_samples"] == 1792 and an["num_classes"] == 10
    assert an["recommendations"]["architecture"] == "lenet"
    cli(["data", "validate", "datasets/mnist", "--num-classes", "10", "--input-shape", "1,28,28"])
    with pytest.raises(SystemExit):
        cli(["data", "validate", "datasets/mnist", "--num-classes", "7"])
    _model_file(ws / "m.axonml")
    cli(["upload", "m.axonml", "--name", "mlp", "--version", "v1", "--validate", "--info"])
    meta = json.load(open("models/mlp-v1.axonml.meta.json"))
    assert meta["parameters"] == 784 * 32 + 32 + 32 * 10 + 10 and meta["format"] == "axonml"
    with pytest.raises(SystemExit):
        cli(["upload", "m.axonml", "--name", "mlp", "--version", "v1"])          # exists, no --overwrite
    cli(["load", "both", "--model", "models/mlp-v1.axonml", "--data", "datasets/mnist"])
    capsys.readouterr()
    cli(["load", "status"])
    out = capsys.readouterr().out
    assert "mlp-v1" in out and "1792 samples" in out
    cli(["analyze", "report", "--format", "json", "--output", "rep.json"])
    rep = json.load(open("rep.json"))
    assert rep["compatibility"] == {"compatible": True, "issues": [], "model_inputs": 784, "model_outputs": 10,
                                    "dataset_features": 784, "dataset_classes": 10}
    cli(["rename", "model", "models/mlp-v1.axonml", "digits"])
    assert os.path.exists("models/digits.axonml") and os.path.exists("models/digits.axonml.meta.json")
    assert json.load(open(".axonml/workspace.json"))["model"]["name"] == "digits"
    cli(["analyze", "model", "--detailed"])
    assert "0.weight" in capsys.readouterr().out
    cli(["load", "clear"])
    with pytest.raises(SystemExit):
        cli(["analyze", "model"])


def test_zip_bundle_roundtrip_and_tabular_data_commands(ws, capsys):
    _model_file(ws / "m.axonml")
    os.makedirs("d")
    with open("d/t.csv", "w") as f:
        f.write("f1,f2,label\n" + "".join(f"{i},{i % 3},{i % 2}\n" for i in range(30)))
    with open("axonml.toml", "w") as f:
        f.write("[project]\nname = 'p'\n")
    cli(["zip", "create", "b.zip", "--model", "m.axonml", "--data", "d", "--include-config"])
    with zipfile.ZipFile("b.zip") as z:
        names = set(z.namelist())
        assert {"model/m.axonml", "dataset/d/t.csv", "config/axonml.toml", "manifest.json"} <= names
        assert json.loads(z.read("manifest.json"))["format"] == "axonml-bundle-v1"
    cli(["zip", "list", "b.zip", "--detailed"])
    assert "dataset/d/t.csv" in capsys.readouterr().out
    cli(["zip", "extract", "b.zip", "--output", "out"])
    assert open("out/model/m.axonml", "rb").read() == open("m.axonml", "rb").read()
    with pytest.raises(SystemExit):
        cli(["zip", "create", "b.zip", "--model", "m.axonml"])
    cli(["data", "config", "d/t.csv", "--output", "gen.toml"])
    import tomllib
    cfg = tomllib.load(open("gen.toml", "rb"))
    assert cfg["model"]["architecture"] == "mlp" and cfg["model"]["num_classes"] == 2 and cfg["model"]["input_size"] == [2]
    cli(["data", "preview", "d/t.csv", "--num-samples", "2"])
    assert "'label': '0'" in capsys.readouterr().out
    cli(["data", "upload", "d", "--name", "toy", "--type", "tabular"])
    cli(["data", "list", "--detailed"])
    assert "toy" in capsys.readouterr().out


def test_scaffold_project_trains(ws):
    cli(["scaffold", "generate", "proj", "--template", "full", "--wandb", "--augment"])
    assert sorted(os.listdir("proj")) == ["README.md", "axonml.toml", "evaluate.py", "infer.py", "output", "train.py"]
    cfg = open("proj/axonml.toml").read().replace("epochs = 10", "epochs = 1")
    open("proj/axonml.toml", "w").write(cfg)
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "train.py"], cwd="proj", env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "epoch 1: loss" in r.stdout and os.path.exists("proj/output/model.axonml")
    runs = os.listdir("proj/wandb")
    assert len(runs) == 1 and runs[0].startswith("offline-run-")
    hist = [json.loads(l) for l in open(f"proj/wandb/{runs[0]}/files/wandb-history.jsonl")]
    assert hist[0]["epoch"] == 1.0 and hist[0]["loss"] > 0
    r = subprocess.run([sys.executable, "evaluate.py"], cwd="proj", env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "accuracy" in r.stdout, r.stderr[-2000:]
    with pytest.raises(SystemExit):
        cli(["scaffold", "generate", "proj"])


def test_wandb_settings_and_offline_run(ws, capsys):
    from axonml_b200.integrations import WandbConfig, WandbRun
    from axonml_b200.integrations.wandb import init_training_run
    cli(["wandb", "config", "--entity", "team", "--project", "vision", "--log-frequency", "2", "--api-key", "k" * 40])
    cli(["wandb", "enable"])
    capsys.readouterr()
    cli(["wandb", "status"])
    out = capsys.readouterr().out
    assert "team" in out and "kkkk" in out and "k" * 40 not in out            # the key is masked
    cfg = WandbConfig.load()
    assert cfg.enabled and cfg.log_frequency == 2 and oct(os.stat(ws / "cfg" / "wandb.json").st_mode)[-3:] == "600"
    run = init_training_run(cfg, "r1", {"lr": 0.1}, directory=str(ws / "wb"))
    assert isinstance(run, WandbRun) and run.url().startswith("https://wandb.ai/team/vision/runs/")
    for i in range(5):
        run.log({"loss": 1.0 / (i + 1)})
    run.summary("best", 0.2)
    d = run.finish()
    rows = [json.loads(l) for l in open(os.path.join(d, "files", "wandb-history.jsonl"))]
    assert [r["_step"] for r in rows] == [0, 1, 2, 3, 4]
    summ = json.load(open(os.path.join(d, "files", "wandb-summary.json")))
    assert summ["best"] == 0.2 and abs(summ["loss"] - 0.2) < 1e-9
    import yaml
    assert yaml.safe_load(open(os.path.join(d, "files", "config.yaml")))["lr"] == {"value": 0.1}
    cli(["wandb", "disable"])
    assert init_training_run(WandbConfig.load(), "r2", {}) is None


def test_kaggle_credentials_and_offline_error(ws):
    from axonml_b200.integrations import KaggleClient, OfflineError
    cli(["kaggle", "login", "someone", "--key", "abc123"])
    k = KaggleClient(timeout=2.0)
    assert k.status()["username"] == "someone" and oct(os.stat(ws / "kaggle" / "kaggle.json").st_mode)[-3:] == "600"
    with pytest.raises(ValueError):
        k.download("not-a-ref")
    try:
        k.search("mnist")
    except OfflineError as e:
        assert "kaggle.com" in str(e)
    os.makedirs(ws / "kaggle" / "datasets" / "owner__set")
    open(ws / "kaggle" / "datasets" / "owner__set" / "a.csv", "w").write("x\n1\n")
    assert k.list_downloaded()[0]["ref"] == "owner/set"
    k.delete_credentials()
    with pytest.raises(PermissionError):
        k.search("x")


def test_tui_renders_every_view(ws):
    from axonml_b200.cli.tui import sparkline
    from axonml_b200.tui import build_app
    _model_file(ws / "m.axonml")
    os.makedirs("output")
    json.dump({"train_loss": [2.0, 1.5, 1.0, 0.7, 0.5]}, open("output/training_history.json", "w"))
    app = build_app("m.axonml")
    text = app.run_once()
    for needle in ("1:Model", "25,450 parameters", "Linear", "[*, 784]", "5 logged", "m.axonml", "next / previous view"):
        assert needle in text, needle
    assert sparkline([1, 2, 3, 4]) == "▁▃▅█" and sparkline([]) == ""
    cli(["tui", "--once", "--model", "m.axonml"])


def test_server_start_status_login_sync_stop(ws, capsys):
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env_pw = "admin-password-1"
    os.environ["AXONML_ADMIN_PASSWORD"] = env_pw
    try:
        cli(["start", "--port", str(port)])
        capsys.readouterr()
        cli(["status", "--format", "json", "--detailed"])
        st = json.loads(capsys.readouterr().out)
        assert st["running"] and st["healthy"] and st["port"] == port and st["health"]["status"] == "healthy"
        with pytest.raises(SystemExit):
            cli(["start", "--port", str(port)])
        cli(["login", "admin@axonml.local", "--password", env_pw, "--server", f"http://127.0.0.1:{port}"])
        assert "logged in" in capsys.readouterr().out
        os.makedirs("models")
        _model_file(ws / "models" / "net.axonml")
        cli(["sync", "--check"])
        assert "would upload models/net.axonml" in capsys.readouterr().out
        cli(["sync"])
        assert "uploaded as version 1" in capsys.readouterr().out
        cli(["sync"])
        assert "to upload: 0" in capsys.readouterr().out
        cli(["logs", "-n", "5"])
        assert "AxonML server and dashboard" in capsys.readouterr().out
        cli(["logout"])
    finally:
        os.environ.pop("AXONML_ADMIN_PASSWORD", None)
        cli(["stop"])
    capsys.readouterr()
    cli(["status"])
    assert "stopped" in capsys.readouterr().out
