"""Training view: progress, per-epoch metrics and timing of a run, followed live from its log.

Parity: crates/axonml-tui/src/views/training.rs (``TrainingStatus``, ``EpochMetrics``,
``TrainingConfig``, ``TrainingSession``; ``TrainingView`` with ``watch_log`` over a file of one JSON
object per line -- keys ``epoch``, ``train_loss``, ``val_loss``, ``train_acc``, ``val_acc``,
``learning_rate``, ``duration_secs`` and the configuration keys ``total_epochs``, ``batch_size``,
``optimizer``, ``model_name`` --, best validation loss, elapsed time and ETA from the mean epoch
time, ``toggle_pause``, ``toggle_details``, ``tick``).  The reference ``tick`` animates demo data;
here it re-reads the log when the file has grown, so a run started with ``axonml train`` is
followed while it writes.  ``{"batch": i, "total_batches": n}`` lines move the batch bar and a
``{"status": ...}`` line ends the run."""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from enum import Enum

from rich.console import Group
from rich.panel import Panel
from rich.progress_bar import ProgressBar
from rich.table import Table
from rich.text import Text

from ..theme import AxonmlTheme as T

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


def format_duration(secs: float | None) -> str:
    if secs is None:
        return "-"
    s = int(secs)
    return f"{s // 3600:d}:{s % 3600 // 60:02d}:{s % 60:02d}" if s >= 3600 else f"{s // 60:d}:{s % 60:02d}"


class TrainingStatus(Enum):
    IDLE = "Idle"
    RUNNING = "Running"
    PAUSED = "Paused"
    COMPLETED = "Completed"
    FAILED = "Failed"

    def style(self) -> str:
        return {"Idle": T.muted(), "Running": T.success(), "Paused": T.warning(), "Completed": T.info(), "Failed": T.error()}[self.value]


@dataclass
class EpochMetrics:
    epoch: int
    train_loss: float
    val_loss: float | None = None
    train_acc: float | None = None
    val_acc: float | None = None
    learning_rate: float = 1e-3
    duration_secs: float = 0.0


@dataclass
class TrainingConfig:
    total_epochs: int = 10
    batch_size: int = 32
    optimizer: str = "Adam"
    initial_lr: float = 1e-3
    model_name: str = "model"


@dataclass
class TrainingSession:
    config: TrainingConfig
    current_epoch: int = 0
    current_batch: int = 0
    total_batches: int = 0
    status: TrainingStatus = TrainingStatus.IDLE
    metrics_history: list = field(default_factory=list)
    best_val_loss: float | None = None
    best_epoch: int | None = None
    elapsed_secs: float = 0.0
    eta_secs: float | None = None


def _num(j: dict, *keys):
    for k in keys:
        v = j.get(k)
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            return float(v)
    return None


def parse_training_log(path: str) -> TrainingSession:
    """Session described by a JSON-lines log, a W&B offline history file or a ``training_history.json``."""
    with open(path) as f:
        content = f.read()
    cfg = TrainingConfig()
    sess = TrainingSession(cfg)
    rows: list[dict] = []
    if path.endswith(".json"):
        j = json.loads(content)
        if isinstance(j, dict):          # lists per metric
            n = max((len(v) for v in j.values() if isinstance(v, list)), default=0)
            rows = [{"epoch": i + 1, **{k: v[i] for k, v in j.items() if isinstance(v, list) and i < len(v)}} for i in range(n)]
            rows.append({k: v for k, v in j.items() if not isinstance(v, list)})
        else:
            rows = [r for r in j if isinstance(r, dict)]
    else:
        for line in content.splitlines():
            line = line.strip()
            if not line:
                continue
            try:
                j = json.loads(line)
            except ValueError:
                continue             # a torn last line while the writer is mid-way
            if isinstance(j, dict):
                rows.append(j)
    by_epoch: dict[int, EpochMetrics] = {}
    final = None
    for j in rows:
        if isinstance(j.get("total_epochs"), int):
            cfg.total_epochs = j["total_epochs"]
        if isinstance(j.get("batch_size"), int):
            cfg.batch_size = j["batch_size"]
        if isinstance(j.get("optimizer"), str):
            cfg.optimizer = j["optimizer"]
        if isinstance(j.get("model_name"), str):
            cfg.model_name = j["model_name"]
        if isinstance(j.get("total_batches"), int):
            sess.total_batches = j["total_batches"]
        if isinstance(j.get("batch"), int):
            sess.current_batch = j["batch"]
        if isinstance(j.get("status"), str):
            final = j["status"].lower()
        ep = j.get("epoch", j.get("_step"))
        loss = _num(j, "train_loss", "loss")
        if isinstance(ep, int) and not isinstance(ep, bool) and loss is not None:
            lr = _num(j, "learning_rate", "lr")
            by_epoch[ep] = EpochMetrics(ep, loss, _num(j, "val_loss"), _num(j, "train_acc", "train_accuracy"),
                                        _num(j, "val_acc", "val_accuracy"), lr if lr is not None else cfg.initial_lr,
                                        _num(j, "duration_secs", "_runtime") or 0.0)
            sess.current_batch = 0
    if not by_epoch:
        raise ValueError("no training metrics found in " + path)
    hist = [by_epoch[k] for k in sorted(by_epoch)]
    cfg.initial_lr = hist[0].learning_rate
    sess.metrics_history = hist
    sess.current_epoch = hist[-1].epoch
    cfg.total_epochs = max(cfg.total_epochs, sess.current_epoch)
    with_val = [m for m in hist if m.val_loss is not None]
    if with_val:
        best = min(with_val, key=lambda m: m.val_loss)
        sess.best_val_loss, sess.best_epoch = best.val_loss, best.epoch
    sess.elapsed_secs = sum(m.duration_secs for m in hist)
    remaining = cfg.total_epochs - sess.current_epoch
    eta = remaining * sess.elapsed_secs / len(hist)
    sess.eta_secs = eta if eta > 0 else None
    if final in ("failed", "error"):
        sess.status = TrainingStatus.FAILED
    elif final in ("completed", "done", "finished") or sess.current_epoch >= cfg.total_epochs:
        sess.status = TrainingStatus.COMPLETED
    return sess


def find_training_log(cwd: str = ".") -> str | None:
    """Newest training log under ``cwd`` (its ``output`` and ``wandb`` trees included)."""
    names = ("training_log.jsonl", "wandb-history.jsonl", "training_history.json")
    cands = []
    for root in (os.path.join(cwd, "output"), os.path.join(cwd, "wandb"), cwd):
        if not os.path.isdir(root):
            continue
        for r, dirs, fs in os.walk(root):
            if r.count(os.sep) - root.count(os.sep) > 4:
                dirs[:] = []
            cands += [os.path.join(r, f) for f in fs if f in names]
    return max(cands, key=os.path.getmtime) if cands else None


class TrainingView:
    LIVE_WINDOW = 30.0      # a log written to within this many seconds belongs to a running job
    VISIBLE = 12

    def __init__(self):
        self.session: TrainingSession | None = None
        self.show_details = True
        self.paused = False
        self.log_path: str | None = None
        self.scroll = 0                  # rows scrolled back from the newest epoch
        self.error = ""
        self._stamp = None

    def watch_log(self, path: str) -> None:
        """Loads ``path`` and follows it from now on; raises when it holds no metrics."""
        sess = parse_training_log(path)
        self.log_path, self.session, self.error = path, sess, ""
        self._stamp = self._file_stamp()
        self._live_status()

    def _file_stamp(self):
        try:
            st = os.stat(self.log_path)
            return (st.st_size, st.st_mtime_ns)
        except OSError:
            return None

    def _live_status(self) -> None:
        s = self.session
        if s is None or s.status in (TrainingStatus.COMPLETED, TrainingStatus.FAILED):
            return
        try:
            fresh = time.time() - os.path.getmtime(self.log_path) < self.LIVE_WINDOW
        except OSError:
            fresh = False
        s.status = TrainingStatus.PAUSED if self.paused else TrainingStatus.RUNNING if fresh else TrainingStatus.IDLE

    def toggle_details(self) -> None:
        self.show_details = not self.show_details

    def toggle_pause(self) -> None:
        """Stops (or resumes) following the log; the job itself is not touched."""
        self.paused = not self.paused
        if not self.paused:
            self.refresh()
        self._live_status()

    def scroll_up(self) -> None:
        if self.session:
            self.scroll = min(self.scroll + 1, max(len(self.session.metrics_history) - self.VISIBLE, 0))

    def scroll_down(self) -> None:
        self.scroll = max(self.scroll - 1, 0)

    def refresh(self) -> bool:
        """Re-reads the log; True when the session changed."""
        if not self.log_path:
            return False
        try:
            self.session = parse_training_log(self.log_path)
            self._stamp = self._file_stamp()
            self.error = ""
        except (OSError, ValueError) as e:
            self.error = str(e)
            return False
        self._live_status()
        return True

    def tick(self) -> bool:
        """Called between key polls: picks up what the job appended since the last read."""
        if self.paused or not self.log_path:
            return False
        if self._file_stamp() != self._stamp:
            return self.refresh()
        before = self.session.status if self.session else None
        self._live_status()
        return bool(self.session) and self.session.status != before

    # ------------------------------------------------------------------ drawing
    def _progress(self) -> Table:
        s = self.session
        g = Table.grid(expand=True, padding=(0, 1))
        g.add_column(width=8, style=T.muted()); g.add_column(ratio=1); g.add_column(width=18, justify="right")
        g.add_row("epochs", ProgressBar(total=max(s.config.total_epochs, 1), completed=s.current_epoch, complete_style=T.success(),
                                        finished_style=T.info()), f"{s.current_epoch}/{s.config.total_epochs}")
        if s.total_batches:
            g.add_row("batches", ProgressBar(total=s.total_batches, completed=min(s.current_batch, s.total_batches),
                                             complete_style=T.accent()), f"{s.current_batch}/{s.total_batches}")
        return g

    def _metrics_table(self) -> Table:
        s = self.session
        tb = Table(expand=True, box=None, pad_edge=False)
        for c in ("epoch", "train loss", "val loss", "train acc", "val acc", "lr", "time"):
            tb.add_column(c, justify="right")
        f = lambda v, p=4: "-" if v is None else f"{v:.{p}f}"
        hist = s.metrics_history
        hi = len(hist) - self.scroll
        for m in hist[max(hi - self.VISIBLE, 0):hi]:
            best = m.epoch == s.best_epoch
            tb.add_row(str(m.epoch), f(m.train_loss), Text(f(m.val_loss) + (" *" if best else ""), style=T.success() if best else ""),
                       f(m.train_acc, 3), f(m.val_acc, 3), f"{m.learning_rate:.2e}", f"{m.duration_secs:.1f}s")
        return tb

    def _details(self) -> Table:
        s = self.session
        last = s.metrics_history[-1]
        tb = Table(box=None, show_header=False, pad_edge=False)
        tb.add_column(style=T.muted()); tb.add_column()
        rows = [("model", s.config.model_name), ("optimizer", s.config.optimizer), ("batch size", str(s.config.batch_size)),
                ("initial lr", f"{s.config.initial_lr:.2e}"), ("current lr", f"{last.learning_rate:.2e}"),
                ("elapsed", format_duration(s.elapsed_secs)), ("ETA", format_duration(s.eta_secs)),
                ("best val loss", "-" if s.best_val_loss is None else f"{s.best_val_loss:.4f} (epoch {s.best_epoch})"),
                ("log", self.log_path or "-")]
        for k, v in rows:
            tb.add_row(k, v)
        return tb

    def render(self):
        if self.session is None:
            msg = self.error or ("no training log found: start a run with `axonml train`, or open a log with --watch <file>")
            return Text(msg, style=T.error() if self.error else T.muted())
        s = self.session
        head = Text.assemble((s.config.model_name, T.title()), "  ", (f"[{s.status.value}]", s.status.style()), "  ",
                             (f"epoch {s.current_epoch}/{s.config.total_epochs}", T.metric_value()), "  ",
                             (f"elapsed {format_duration(s.elapsed_secs)}", T.muted()), "  ", (f"ETA {format_duration(s.eta_secs)}", T.muted()))
        losses = [m.train_loss for m in s.metrics_history]
        spark = Text.assemble(("loss ", T.muted()), (sparkline(losses), T.series(0)), (f"  {losses[0]:.4g} -> {losses[-1]:.4g}", T.muted()))
        body = [head, self._progress(), spark]
        table = Panel(self._metrics_table(), title=f"Epochs ({len(s.metrics_history)} logged)", border_style=T.border_focused())
        if self.show_details:
            grid = Table.grid(expand=True)
            grid.add_column(ratio=3); grid.add_column(ratio=2)
            grid.add_row(table, Panel(self._details(), title="Run", border_style=T.border()))
            body.append(grid)
        else:
            body.append(table)
        if self.error:
            body.append(Text(self.error, style=T.error()))
        return Group(*body)
