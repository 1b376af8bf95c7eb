"""The example programs (the reference ships six under crates/axonml/examples and one under
crates/axonml-core/examples) run end to end on the CPU."""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture()
def examples(monkeypatch, tmp_path):
    monkeypatch.syspath_prepend(os.path.join(ROOT, "examples"))
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    for m in ("simple_training", "mnist_training", "hvac_model", "hvac_training", "hvac_inference", "nlp_audio_test", "gpu_test"):
        sys.modules.pop(m, None)
    return lambda name: importlib.import_module(name)


def test_simple_training_learns_xor(examples):
    assert examples("simple_training").main(epochs=400) < 0.02


def test_mnist_training_on_the_synthetic_set(examples):
    acc = examples("mnist_training").main(["--epochs", "2", "--samples", "512", "--device", "cpu", "--data", "nowhere"])
    assert acc > 0.5


def test_hvac_model_training_and_inference(examples, tmp_path):
    model = examples("hvac_model").main()
    assert sum(p.numel() for p in model.parameters()) == 280_316
    accs = examples("hvac_training").main(["--epochs", "1", "--scenarios", "14", "--length", "300", "--device", "cpu",
                                           "--output", str(tmp_path / "hvac.axonml")])
    assert len(accs) == 3 and all(0.0 <= a <= 1.0 for a in accs)
    out = examples("hvac_inference").main(str(tmp_path / "hvac.axonml"))
    assert set(out) == {"5 min", "15 min", "30 min"} and abs(sum(v for _, v in out["5 min"])) <= 1.0 + 1e-5


def test_nlp_audio_tour(examples):
    r = examples("nlp_audio_test").main()
    assert r["encoded"] == [5, 6, 8] and r["resampled"] == 4000 and r["mel"] == (40, 51) and r["mfcc"] == (13, 51)
    assert 18.0 < r["snr_db"] < 22.0 and abs(r["peak"] - 1.0) < 1e-4


def test_gpu_test_example_without_a_device(examples):
    assert examples("gpu_test").main() == 0


def test_context_parallel_example_single_process(examples, monkeypatch):
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    sys.modules.pop("context_parallel_llama", None)
    first = examples("context_parallel_llama").main("ulysses", steps=1)
    sys.modules.pop("context_parallel_llama", None)
    assert examples("context_parallel_llama").main("ring", steps=8) < first
