"""Terminal user interface: Model / Data / Training / Graphs / Files / Help views with vim-style
keys, rendered with ``rich``.

Parity: crates/axonml-tui (``app.rs`` tab set and key map: 1-6 or Tab to switch views, j/k to move,
Enter to open, r to refresh, ? for help, q to quit; ``views/*.rs``).  The reference draws with
ratatui on a crossterm raw-mode terminal; here each frame is a ``rich`` layout printed to the
terminal, and keys are read in cbreak mode when stdin is a TTY.  ``run_once`` renders every view to
a string, which is what the tests and ``axonml tui --once`` use."""
from __future__ import annotations

import json
import os
import sys

from rich.console import Console, Group
from rich.panel import Panel
from rich.table import Table
from rich.text import Text

VIEWS = ["Model", "Data", "Training", "Graphs", "Files", "Help"]
KEYS = [("1-6 / Tab", "switch view"), ("j / k", "move down / up"), ("Enter", "open the selected file"), ("r", "refresh"),
        ("?", "help"), ("q", "quit")]
_SPARK = " ▁▂▃▄▅▆▇█"


def sparkline(values, width: int = 60) -> str:
    vals = [v for v in values if v is not None]
    if not vals:
        return ""
    if len(vals) > width:
        step = len(vals) / width
        vals = [vals[int(i * step)] for i in range(width)]
    lo, hi = min(vals), max(vals)
    return "".join(_SPARK[1 + int((v - lo) / (hi - lo or 1) * (len(_SPARK) - 2))] for v in vals)


class TuiApp:
    def __init__(self, model: str | None = None, data: str | None = None, cwd: str = "."):
        self.model_path, self.data_path, self.cwd = model, data, cwd
        self.view, self.cursor, self.message = 0, 0, ""
        self._model = self._data = None
        self.refresh()

    # ------------------------------------------------------------------ state
    def refresh(self) -> None:
        from .workspace import _ws_load, model_summary
        ws = _ws_load()
        mp = self.model_path or (ws["model"]["path"] if ws.get("model") else None)
        dp = self.data_path or (ws["dataset"]["path"] if ws.get("dataset") else None)
        self._model = self._data = None
        try:
            if mp:
                self._model = model_summary(mp)
            if dp:
                from ..data.analysis import analyze_dataset
                self._data = analyze_dataset(dp, max_samples=2000)
        except Exception as e:  # noqa: BLE001 - shown in the status line
            self.message = f"{type(e).__name__}: {e}"
        self.files = sorted(f for f in os.listdir(self.cwd) if not f.startswith("."))[:200]
        self.history = self._load_history()

    def _load_history(self) -> list[dict]:
        """Loss points of the newest offline W&B run or ``training_history.json`` under the cwd."""
        cands = []
        for root in (os.path.join(self.cwd, "wandb"), os.path.join(self.cwd, "output"), self.cwd):
            if os.path.isdir(root):
                for r, _, fs in os.walk(root):
                    for f in fs:
                        if f in ("wandb-history.jsonl", "training_history.json"):
                            cands.append(os.path.join(r, f))
        if not cands:
            return []
        path = max(cands, key=os.path.getmtime)
        try:
            with open(path) as f:
                if path.endswith(".jsonl"):
                    return [json.loads(l) for l in f if l.strip()]
                j = json.load(f)
                return j if isinstance(j, list) else [{"loss": v, "_step": i} for i, v in enumerate(j.get("train_loss", []))]
        except (OSError, ValueError):
            return []

    def key(self, k: str) -> bool:
        """Applies one key; False means quit."""
        if k == "q":
            return False
        if k in "123456":
            self.view, self.cursor = int(k) - 1, 0
        elif k == "\t":
            self.view, self.cursor = (self.view + 1) % len(VIEWS), 0
        elif k == "?":
            self.view = VIEWS.index("Help")
        elif k == "j":
            self.cursor += 1
        elif k == "k":
            self.cursor = max(0, self.cursor - 1)
        elif k == "r":
            self.refresh()
            self.message = "refreshed"
        elif k in ("\r", "\n") and VIEWS[self.view] == "Files" and self.files:
            f = os.path.join(self.cwd, self.files[min(self.cursor, len(self.files) - 1)])
            if f.endswith((".axonml", ".safetensors", ".gguf", ".onnx")):
                self.model_path, self.view = f, 0
            elif os.path.isdir(f) or f.endswith((".csv", ".tsv")):
                self.data_path, self.view = f, 1
            self.refresh()
        return True

    # ------------------------------------------------------------------ views
    def _tabs(self) -> Text:
        t = Text()
        for i, v in enumerate(VIEWS):
            t.append(f" {i + 1}:{v} ", style="bold black on cyan" if i == self.view else "cyan")
        return t

    def _view_model(self):
        m = self._model
        if not m:
            return Text("no model loaded  (axonml load model <path>, or open one from the Files view)", style="dim")
        tb = Table(title=f"{os.path.basename(m['path'])}: {m['format']}, {m['parameters']:,} parameters, {m['file_bytes']:,} bytes")
        tb.add_column("layer"); tb.add_column("parameters", justify="right")
        rows = m["layers"]
        lo = min(self.cursor, max(len(rows) - 1, 0))
        for i, l in enumerate(rows[lo:lo + 25]):
            tb.add_row(l["name"], f"{l['parameters']:,}", style="reverse" if i == 0 else None)
        return tb

    def _view_data(self):
        d = self._data
        if not d:
            return Text("no dataset loaded  (axonml load data <path>)", style="dim")
        tb = Table(title=f"{d['path']}: {d['dataset_type']}, {d.get('num_samples')} samples, {d.get('num_classes')} classes")
        tb.add_column("class"); tb.add_column("count", justify="right"); tb.add_column("share")
        cc = d.get("class_counts") or {}
        tot = sum(cc.values()) or 1
        for k, v in sorted(cc.items(), key=lambda kv: -kv[1])[:20]:
            tb.add_row(str(k), str(v), "█" * int(30 * v / tot))
        rec = d.get("recommendations", {})
        return Group(tb, Text("recommended: " + ", ".join(f"{k}={v}" for k, v in rec.items() if k != "notes")))

    def _view_training(self):
        h = self.history
        if not h:
            return Text("no training history found under ./wandb or ./output", style="dim")
        tb = Table(title=f"{len(h)} logged points")
        keys = [k for k in h[-1] if not k.startswith("_")][:6]
        tb.add_column("step", justify="right")
        for k in keys:
            tb.add_column(k, justify="right")
        for row in h[-12:]:
            tb.add_row(str(row.get("_step", "")), *[f"{row.get(k):.4g}" if isinstance(row.get(k), (int, float)) else "" for k in keys])
        return tb

    def _view_graphs(self):
        h = self.history
        if not h:
            return Text("nothing to plot yet", style="dim")
        out = []
        for k in [k for k in h[-1] if not k.startswith("_")][:4]:
            vals = [r.get(k) for r in h if isinstance(r.get(k), (int, float))]
            if vals:
                out.append(Text(f"{k:12s} {sparkline(vals)}  {vals[0]:.4g} -> {vals[-1]:.4g}"))
        return Group(*out)

    def _view_files(self):
        tb = Table(title=os.path.abspath(self.cwd))
        tb.add_column("name"); tb.add_column("bytes", justify="right")
        cur = min(self.cursor, max(len(self.files) - 1, 0))
        lo = max(0, cur - 12)
        for i, f in enumerate(self.files[lo:lo + 25]):
            p = os.path.join(self.cwd, f)
            tb.add_row(f + ("/" if os.path.isdir(p) else ""), "" if os.path.isdir(p) else f"{os.path.getsize(p):,}",
                       style="reverse" if lo + i == cur else None)
        return tb

    def _view_help(self):
        tb = Table(title="keys")
        tb.add_column("key"); tb.add_column("action")
        for k, v in KEYS:
            tb.add_row(k, v)
        return tb

    def render(self):
        body = getattr(self, "_view_" + VIEWS[self.view].lower())()
        return Group(self._tabs(), Panel(body, title=f"AxonML - {VIEWS[self.view]}", border_style="cyan"),
                     Text(self.message or "q quit   ? help   1-6 views", style="dim"))

    def run_once(self, width: int = 110) -> str:
        """Every view rendered once, as plain text."""
        con = Console(width=width, record=True, file=open(os.devnull, "w"), force_terminal=False)
        for i in range(len(VIEWS)):
            self.view = i
            con.print(self.render())
        return con.export_text()

    def run(self) -> None:
        con = Console()
        if not sys.stdin.isatty():
            con.print(self.render())
            return
        import termios
        import tty
        fd = sys.stdin.fileno()
        old = termios.tcgetattr(fd)
        try:
            tty.setcbreak(fd)
            while True:
                con.clear()
                con.print(self.render())
                self.message = ""
                if not self.key(sys.stdin.read(1)):
                    break
        finally:
            termios.tcsetattr(fd, termios.TCSADRAIN, old)


def cmd_tui(a) -> None:
    app = TuiApp(a.model, a.data)
    if a.once:
        print(app.run_once())
    else:
        app.run()
