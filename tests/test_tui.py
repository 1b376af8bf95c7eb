"""Terminal interface: key decoding, key map, the six views on real files, and following a log.

Mirrors the reference's tests of crates/axonml-tui (app.rs / event.rs: tab cycling, direct tab
keys, quit, help overlay closed by any key) and adds the parts that are demo data there: model and
dataset analysis, the file tree and the live training log."""
import json
import os

import pytest
import torch

from axonml_b200.tui import App, StatusLevel, Tab, build_app
from axonml_b200.tui import keys as K
from axonml_b200.tui.views import (BrailleCanvas, ChartType, FilesView, FileType, GraphsView, TrainingStatus, TrainingView,
                                   find_training_log, parse_training_log)
from axonml_b200.tui.views.graphs import DataSeries, plot
from axonml_b200.tui.views.model import classify_layer, format_count, format_size, model_info


@pytest.fixture()
def ws(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("AXONML_HOME", str(tmp_path / "home"))
    monkeypatch.setenv("AXONML_CONFIG_DIR", str(tmp_path / "cfg"))
    return tmp_path


def _model_file(path):
    from axonml_b200 import nn
    from axonml_b200.serialize import save_state_dict
    from axonml_b200.serialize.state_dict import StateDict
    torch.manual_seed(0)
    net = nn.Sequential(nn.Conv2d(3, 8, 3), nn.BatchNorm2d(8), nn.ReLU(), nn.Identity(), nn.Linear(8 * 6 * 6, 16), nn.LayerNorm(16),
                        nn.Linear(16, 4))
    save_state_dict(StateDict.from_module(net), str(path))
    return sum(p.numel() for p in net.parameters())


def _log(path, epochs, total=6, status=None):
    with open(path, "w") as f:
        f.write(json.dumps({"model_name": "lenet", "total_epochs": total, "batch_size": 64, "optimizer": "adamw", "total_batches": 40}) + "\n")
        for e in range(1, epochs + 1):
            f.write(json.dumps({"epoch": e, "train_loss": 2.0 / e, "val_loss": 2.2 / e + (0.3 if e == epochs and e > 2 else 0.0),
                                "train_acc": 0.5 + 0.05 * e, "val_acc": 0.45 + 0.05 * e, "learning_rate": 1e-3 * 0.9 ** e,
                                "duration_secs": 10.0}) + "\n")
        if status:
            f.write(json.dumps({"status": status}) + "\n")


def test_key_decoder_handles_control_bytes_and_escape_sequences():
    assert K.decode(b"jk") == ["j", "k"]
    assert K.decode(b"\x1b[A\x1b[B\x1b[C\x1b[D") == [K.UP, K.DOWN, K.RIGHT, K.LEFT]
    assert K.decode(b"\x1bOA") == [K.UP]                                  # application cursor mode
    assert K.decode(b"\x1b[Z\t\r\x7f") == [K.BACKTAB, K.TAB, K.ENTER, K.BACKSPACE]
    assert K.decode(b"\x1b[5~\x1b[6~\x1b[H\x1b[F") == [K.PAGE_UP, K.PAGE_DOWN, K.HOME, K.END]
    assert K.decode(b"\x1b[1;5A") == [K.UP]                               # modifiers are ignored
    assert K.decode(b"\x1b") == [K.ESC] and K.decode(b"\x03") == ["q"]
    assert K.decode("~é".encode()) == ["~", "é"] and K.decode(b"\x00\x01") == []


def test_tabs_cycle_and_global_keys(ws):
    app = App()
    assert app.active_tab is Tab.MODEL and not app.should_quit
    assert [t.key() for t in Tab.all()] == ["1", "2", "3", "4", "5", "?"]
    assert Tab.MODEL.prev() is Tab.HELP and Tab.HELP.next() is Tab.MODEL
    app.handle_key(K.TAB)
    assert app.active_tab is Tab.DATA
    app.handle_key(K.BACKTAB); app.handle_key(K.BACKTAB)
    assert app.active_tab is Tab.HELP
    for k, tab in zip("12345", Tab.all()):
        app.handle_key(k)
        assert app.active_tab is tab
    app.handle_key("?")
    assert app.show_help and "next / previous view" in app.frame()
    app.handle_key("q")                                                  # any key only closes the overlay
    assert not app.show_help and not app.should_quit and app.active_tab is Tab.FILES
    app.handle_key("q")
    assert app.should_quit


def test_status_line_reports_and_expires(ws):
    app = App()
    app.set_status("saved", StatusLevel.SUCCESS)
    assert "saved" in app.frame()
    app.status.at -= App.STATUS_SECONDS + 1
    assert app.tick() and app.status is None and "q quit" in app.frame()
    assert not app.load_model("missing.axonml") and app.status.level is StatusLevel.ERROR
    assert "missing.axonml" in app.frame()


def test_model_view_infers_layer_kinds_and_navigates(ws):
    n = _model_file(ws / "net.axonml")
    info = model_info("net.axonml")
    kinds = {l.name: l.layer_type for l in info.layers}
    assert kinds == {"0": "Conv2d", "1": "BatchNorm", "4": "Linear", "5": "LayerNorm", "6": "Linear"}
    assert info.trainable_params == n and info.total_params == n and info.format == "axonml"
    conv = info.layers[0]
    assert conv.input_shape == "[N, 3, H, W]" and conv.params == 3 * 8 * 9 + 8 and conv.bytes == 4 * conv.params
    assert ("weight", [8, 3, 3, 3], "float32") in conv.tensors
    assert classify_layer("model.embed_tokens", {"weight": [100, 16]})[0] == "Embedding"
    assert classify_layer("norm", {"weight": [16]})[0] == "RMSNorm"
    assert classify_layer("conv", {"weight": [4, 2, 5], "bias": [4]})[0] == "Conv1d"
    assert format_count(1_250_000) == "1.25M" and format_count(999) == "999" and format_size(3 << 20) == "3.0 MB"
    app = App()
    assert app.load_model("net.axonml") and app.active_tab is Tab.MODEL and app.status.level is StatusLevel.SUCCESS
    text = app.frame()
    for needle in ("Conv2d", "BatchNorm", "LayerNorm", f"{n:,} parameters", "Details", "8x3x3x3", "of the model"):
        assert needle in text, needle
    app.handle_key("j"); app.handle_key(K.DOWN)
    assert app.model_view.selected_layer == 2 and "288" in app.frame()
    for _ in range(9):
        app.handle_key("j")
    assert app.model_view.selected_layer == 4
    app.handle_key(K.PAGE_UP)
    assert app.model_view.selected_layer == 0
    app.handle_key("d")
    assert not app.model_view.show_details and "Details" not in app.frame()
    app.handle_key(K.ENTER)
    assert app.model_view.show_details


def test_data_view_on_a_table(ws):
    rows = ["a,b,label"] + [f"{i},{i * 0.5},{'cat' if i % 4 else 'dog'}" for i in range(40)]
    (ws / "pets.csv").write_text("\n".join(rows) + "\n")
    app = App()
    assert app.load_dataset("pets.csv") and app.active_tab is Tab.DATA
    d = app.data_view.dataset
    assert d.total_samples == 40 and d.num_classes == 2 and d.feature_dim == "2"
    assert [(c.name, c.count) for c in d.classes] == [("cat", 30), ("dog", 10)] and d.classes[0].percentage == 75.0
    assert [f.name for f in d.features] == ["a", "b", "label"] and d.features[1].max == 19.5 and d.features[2].dtype == "categorical"
    assert [(s.name, s.samples) for s in d.splits] == [("train", 32), ("validation", 8)]
    text = app.frame()
    for needle in ("pets.csv", "40 samples", "75.0%", "19.5", "train 32 (80%)", "recommended: batch_size=16"):
        assert needle in text, needle
    app.handle_key("j")
    assert app.data_view.selected_class == 1
    app.handle_key("j")
    assert app.data_view.selected_class == 1                              # clamps at the last class
    app.handle_key("l"); app.handle_key("j"); app.handle_key("j"); app.handle_key("j")
    assert app.data_view.active_panel == 1 and app.data_view.selected_feature == 2
    app.handle_key(K.LEFT)
    assert app.data_view.active_panel == 0


def test_data_view_uses_split_folders_of_an_image_dataset(ws):
    for split, n in (("train", 6), ("val", 2), ("test", 1)):
        for cls in ("ants", "bees"):
            os.makedirs(ws / "insects" / split / cls)
            for i in range(n):
                (ws / "insects" / split / cls / f"{i}.png").write_bytes(b"\x89PNG")
    app = App()
    assert app.load_dataset("insects")
    assert {s.name: s.samples for s in app.data_view.dataset.splits} == {"train": 12, "validation": 4, "test": 2}


def test_training_log_parsing(ws):
    _log("run.jsonl", 4)
    with open("run.jsonl", "a") as f:
        f.write('{"epoch": 5, "train_lo')                               # a torn line is skipped
    s = parse_training_log("run.jsonl")
    assert s.config.model_name == "lenet" and s.config.total_epochs == 6 and s.config.optimizer == "adamw" and s.config.batch_size == 64
    assert s.current_epoch == 4 and len(s.metrics_history) == 4 and s.total_batches == 40
    assert s.best_epoch == 3 and s.best_val_loss == pytest.approx(2.2 / 3)       # epoch 4 carries the penalty
    assert s.elapsed_secs == 40.0 and s.eta_secs == 20.0 and s.status is TrainingStatus.IDLE
    assert s.config.initial_lr == pytest.approx(9e-4)
    _log("done.jsonl", 6)
    assert parse_training_log("done.jsonl").status is TrainingStatus.COMPLETED and parse_training_log("done.jsonl").eta_secs is None
    _log("bad.jsonl", 2, status="failed")
    assert parse_training_log("bad.jsonl").status is TrainingStatus.FAILED
    (ws / "empty.jsonl").write_text('{"total_epochs": 3}\n')
    with pytest.raises(ValueError):
        parse_training_log("empty.jsonl")
    # the offline W&B history and the per-metric lists of training_history.json are read too
    (ws / "wandb-history.jsonl").write_text('{"_step": 1, "train_loss": 1.0, "val_accuracy": 0.5}\n{"_step": 2, "train_loss": 0.5, "val_accuracy": 0.7}\n')
    w = parse_training_log("wandb-history.jsonl")
    assert [m.val_acc for m in w.metrics_history] == [0.5, 0.7]
    json.dump({"train_loss": [3.0, 2.0, 1.0], "val_loss": [3.5, 2.5]}, open("training_history.json", "w"))
    h = parse_training_log("training_history.json")
    assert [m.train_loss for m in h.metrics_history] == [3.0, 2.0, 1.0] and h.metrics_history[2].val_loss is None and h.best_epoch == 2


def test_training_view_follows_a_growing_log(ws):
    os.makedirs("output")
    _log("output/training_log.jsonl", 2)
    assert find_training_log(".") == os.path.join(".", "output", "training_log.jsonl")
    app = build_app()
    assert app.training_view.session.current_epoch == 2 and app.active_tab is Tab.MODEL
    assert app.training_view.session.status is TrainingStatus.RUNNING           # written to a moment ago
    app.handle_key("3")
    text = app.frame()
    for needle in ("lenet", "[Running]", "epoch 2/6", "2/6", "0/40", "adamw", "ETA 0:40", "best val loss", "1.1000 (epoch 2)"):
        assert needle in text, needle
    assert not app.tick()                                                # nothing new
    _log("output/training_log.jsonl", 5)
    assert app.tick() and app.training_view.session.current_epoch == 5
    assert len(app.graphs_view.train_loss) == 5                          # the Graphs view got the new points
    app.handle_key("p")
    assert app.training_view.paused and app.training_view.session.status is TrainingStatus.PAUSED and "[Paused]" in app.frame()
    _log("output/training_log.jsonl", 6, status="completed")
    assert not app.tick() and app.training_view.session.current_epoch == 5       # paused: not followed
    app.handle_key("p")
    assert app.training_view.session.current_epoch == 6 and app.training_view.session.status is TrainingStatus.COMPLETED
    assert "[Completed]" in app.frame()
    app.handle_key("d")
    assert "optimizer" not in app.frame()
    tv = TrainingView()
    tv.VISIBLE = 3
    tv.watch_log("output/training_log.jsonl")
    tv.scroll_up(); tv.scroll_up(); tv.scroll_up(); tv.scroll_up()
    assert tv.scroll == 3
    tv.scroll_down()
    assert tv.scroll == 2
    # an old log belongs to no running job
    _log("old.jsonl", 2)
    os.utime("old.jsonl", (1, 1))
    tv.watch_log("old.jsonl")
    assert tv.session.status is TrainingStatus.IDLE


def test_graphs_view_charts_zoom_and_canvas(ws):
    cv = BrailleCanvas(2, 1)
    cv.set(0, 0, "red"); cv.set(1, 3, "red"); cv.set(3, 0, "blue"); cv.set(99, 99, "x")
    assert [str(r) for r in cv.rows()] == ["\u2881\u2808"]
    cv = BrailleCanvas(3, 1)
    cv.line(0, 3, 5, 0, "")
    assert all(b for b in cv.bits[0])                                    # the line crosses every cell
    rows = plot([DataSeries("s", [(0.0, 0.0), (10.0, 1.0)], "")], (0.0, 10.0), (0.0, 1.0), width=20, height=4)
    assert len(rows) == 6 and "1.000" in str(rows[0]) and "0.000" in str(rows[3]) and str(rows[5]).strip().startswith("0")
    _log("run.jsonl", 6)
    g = GraphsView()
    assert "nothing to plot" in _text(g.render())
    g.set_session(parse_training_log("run.jsonl"))
    assert g.x_bounds == [1.0, 6.0] and g.loss_bounds[0] == 0.0 and g.loss_bounds[1] == pytest.approx(2.2 * 1.05)
    assert g.acc_bounds == [0.0, 1.0] and g.active_chart is ChartType.LOSS
    t = _text(g.render())
    assert "train loss (last 0.3333)" in t and "validation loss" in t and "Loss by epoch" in t
    g.next_chart()
    assert g.active_chart is ChartType.ACCURACY and "validation accuracy (last 0.75)" in _text(g.render())
    g.next_chart()
    assert g.active_chart is ChartType.LEARNING_RATE and "e-0" in _text(g.render())     # small values use exponents
    g.next_chart(); g.prev_chart()
    assert g.active_chart is ChartType.LEARNING_RATE
    g.prev_chart(); g.prev_chart(); g.toggle_zoom()
    xb, yb = g.bounds()
    assert xb == [3.5, 6.0] and yb[1] < 1.0 and "zoom" in _text(g.render())
    app = App()
    app.watch_training("run.jsonl")
    app.handle_key("4"); app.handle_key("l"); app.handle_key("z")
    assert app.graphs_view.active_chart is ChartType.ACCURACY and app.graphs_view.zoomed and "Accuracy by epoch" in app.frame()


def _text(renderable) -> str:
    from rich.console import Console
    with open(os.devnull, "w") as sink:
        con = Console(width=120, record=True, file=sink, color_system=None)
        con.print(renderable)
        return con.export_text()


def test_files_view_tree_preview_and_opening(ws):
    _model_file(ws / "net.axonml")
    os.makedirs(ws / "data" / "raw")
    (ws / "data" / "pets.csv").write_text("a,label\n1,x\n2,y\n")
    (ws / "data" / "raw" / "notes.txt").write_text("first line\nsecond line\n")
    (ws / "axonml.toml").write_text("[project]\nname = \"demo\"\n")
    (ws / ".secret").write_text("x")
    _log("training_log.jsonl", 3)
    assert FileType.from_extension(".SafeTensors") is FileType.MODEL and FileType.from_extension("parquet") is FileType.DATASET
    assert FileType.from_extension("yml") is FileType.CONFIG and FileType.from_extension("rs") is FileType.OTHER
    app = App()
    v = app.files_view
    assert [e.name for e in v.entries] == ["data", "axonml.toml", "net.axonml", "training_log.jsonl"]      # folders first, dot files hidden
    assert v.entries[0].file_type is FileType.DIRECTORY and v.entries[2].file_type is FileType.MODEL
    app.handle_key("5")
    app.handle_key(K.ENTER)                                              # expands data/ in place
    assert [e.name for e in v.entries][:3] == ["data", "raw", "pets.csv"] and v.entries[1].depth == 1 and v.entries[0].is_expanded
    assert "▾ data/" in app.frame() and "Entries: 2" in app.frame()
    app.handle_key("j"); app.handle_key(K.ENTER); app.handle_key("j")
    assert v.entries[v.selected].name == "notes.txt" and v.entries[v.selected].depth == 2 and "second line" in v.preview
    app.handle_key("j")
    assert v.entries[v.selected].name == "pets.csv"
    app.handle_key(K.ENTER)
    assert app.active_tab is Tab.DATA and app.data_view.dataset.total_samples == 2
    app.handle_key("5")
    app.handle_key(K.ENTER)                                              # selection is kept: pets.csv again
    app.handle_key("5")
    app.handle_key("k"); app.handle_key("k"); app.handle_key("k"); app.handle_key(K.ENTER)      # collapses data/
    assert [e.name for e in v.entries] == ["data", "axonml.toml", "net.axonml", "training_log.jsonl"]
    app.handle_key("j")
    assert 'name = "demo"' in v.preview                                  # config files are previewed as text
    app.handle_key(K.ENTER)
    assert app.active_tab is Tab.FILES and "previewed only" in app.status.text
    app.handle_key("j"); app.handle_key(K.ENTER)
    assert app.active_tab is Tab.MODEL and app.model_view.model.name == "net.axonml"
    app.handle_key("5"); app.handle_key("j"); app.handle_key(K.ENTER)
    assert app.active_tab is Tab.TRAINING and app.training_view.session.current_epoch == 3
    app.handle_key("5"); app.handle_key(".")
    assert v.show_hidden and ".secret" in [e.name for e in v.entries]
    app.handle_key(".")
    v.set_filter("TOML")
    assert [e.name for e in v.entries] == ["data", "axonml.toml"]
    v.set_filter(None)
    v.selected = 0
    app.handle_key("l")                                                  # data/ becomes the root
    assert v.current_dir == str(ws / "data") and [e.name for e in v.entries] == ["raw", "notes.txt", "pets.csv"]      # raw/ stays expanded
    app.handle_key("u")
    assert v.current_dir == str(ws) and v.entries[v.selected].name == "data"      # back on the folder we came from
    app.handle_key("o")
    assert app.active_tab is Tab.DATA                                    # a folder opened as a dataset
    v.go_home()
    assert v.current_dir == os.path.expanduser("~")


def test_train_command_writes_the_log_the_interface_follows(ws, capsys):
    from axonml_b200.cli.main import main as cli
    cli(["new", "demo"])
    os.chdir("demo")
    cli(["train", "--epochs", "2", "--device", "cpu"])
    capsys.readouterr()
    s = parse_training_log("output/training_log.jsonl")
    assert s.status is TrainingStatus.COMPLETED and s.current_epoch == 2 and s.config.total_epochs == 2 and s.total_batches > 0
    assert all(m.duration_secs > 0 and m.learning_rate > 0 for m in s.metrics_history)
    cli(["tui", "--once", "--watch", "output/training_log.jsonl"])
    out = capsys.readouterr().out
    assert "[Completed]" in out and "Loss by epoch" in out
