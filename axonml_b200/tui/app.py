"""Application state, key handling and the draw loop of the terminal interface.

Parity: crates/axonml-tui/src/app.rs (``App`` holding the six views, ``Tab`` with ``all`` / ``name``
/ ``key`` / ``next`` / ``prev``, ``StatusMessage`` + ``StatusLevel``, ``load_model`` /
``load_dataset`` / ``watch_training`` which report through the status line and switch tab, ``quit``),
src/event.rs (``handle_key_event``: global keys first -- q, ?, Tab / BackTab, 1-5 --, any key closes
the help overlay, then the active view's own keys) and src/ui.rs / src/lib.rs (header with the tab
bar, body, footer with the status line; ``run`` with a 100 ms poll that also ticks the Training
view).  Drawing goes through ``rich`` instead of ratatui; ``App.frame()`` returns one frame as text,
which is what the tests and ``axonml tui --once`` print."""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass
from enum import Enum

from rich.console import Console, Group
from rich.panel import Panel
from rich.text import Text

from . import keys as K
from .theme import AxonmlTheme as T
from .views import DataView, FilesView, GraphsView, HelpView, ModelView, TrainingView, find_training_log
from .views.files import FileType

_MODEL_EXT = (".axonml", ".onnx", ".safetensors", ".st", ".pt", ".pth", ".gguf", ".bin")
_DATA_EXT = (".npz", ".csv", ".tsv", ".parquet", ".idx", "-ubyte")
_LOG_NAMES = ("training_log.jsonl", "wandb-history.jsonl", "training_history.json")


class Tab(Enum):
    MODEL = "Model"
    DATA = "Data"
    TRAINING = "Training"
    GRAPHS = "Graphs"
    FILES = "Files"
    HELP = "Help"

    @classmethod
    def all(cls) -> list:
        return list(cls)

    def name_(self) -> str:
        return self.value

    def key(self) -> str:
        return "?" if self is Tab.HELP else str(Tab.all().index(self) + 1)

    def next(self) -> "Tab":
        order = Tab.all()
        return order[(order.index(self) + 1) % len(order)]

    def prev(self) -> "Tab":
        order = Tab.all()
        return order[(order.index(self) - 1) % len(order)]


class StatusLevel(Enum):
    INFO = "info"
    SUCCESS = "success"
    WARNING = "warning"
    ERROR = "error"


@dataclass
class StatusMessage:
    text: str
    level: StatusLevel
    at: float


class App:
    STATUS_SECONDS = 6.0

    def __init__(self, cwd: str = "."):
        self.active_tab = Tab.MODEL
        self.should_quit = False
        self.show_help = False
        self.status: StatusMessage | None = None
        self.model_view, self.data_view = ModelView(), DataView()
        self.training_view, self.graphs_view = TrainingView(), GraphsView()
        self.files_view, self.help_view = FilesView(cwd), HelpView()
        self.cwd = cwd

    # ------------------------------------------------------------------ state changes
    def next_tab(self) -> None: self.active_tab = self.active_tab.next()
    def prev_tab(self) -> None: self.active_tab = self.active_tab.prev()
    def go_to_tab(self, tab: Tab) -> None: self.active_tab = tab
    def toggle_help(self) -> None: self.show_help = not self.show_help
    def quit(self) -> None: self.should_quit = True

    def set_status(self, text: str, level: StatusLevel = StatusLevel.INFO) -> None:
        self.status = StatusMessage(text, level, time.monotonic())

    def clear_status(self) -> None:
        self.status = None

    def load_model(self, path: str) -> bool:
        try:
            self.model_view.load_model(path)
        except Exception as e:  # noqa: BLE001 - any reader error is shown, the interface stays up
            self.model_view.error = f"{os.path.basename(path)}: {type(e).__name__}: {e}"
            self.set_status(f"could not load model {path}: {e}", StatusLevel.ERROR)
            return False
        m = self.model_view.model
        self.set_status(f"loaded model {m.name}: {len(m.layers)} layers, {m.total_params:,} parameters", StatusLevel.SUCCESS)
        self.go_to_tab(Tab.MODEL)
        return True

    def load_dataset(self, path: str) -> bool:
        try:
            self.data_view.load_dataset(path)
        except Exception as e:  # noqa: BLE001
            self.data_view.error = f"{os.path.basename(path)}: {type(e).__name__}: {e}"
            self.set_status(f"could not load dataset {path}: {e}", StatusLevel.ERROR)
            return False
        d = self.data_view.dataset
        self.set_status(f"loaded dataset {d.name}: {d.total_samples:,} samples, {d.num_classes} classes", StatusLevel.SUCCESS)
        self.go_to_tab(Tab.DATA)
        return True

    def watch_training(self, path: str) -> bool:
        try:
            self.training_view.watch_log(path)
        except (OSError, ValueError) as e:
            self.training_view.error = str(e)
            self.set_status(f"could not read training log {path}: {e}", StatusLevel.ERROR)
            return False
        self.graphs_view.set_session(self.training_view.session)
        self.set_status(f"watching {path}", StatusLevel.INFO)
        self.go_to_tab(Tab.TRAINING)
        return True

    def load_workspace(self) -> None:
        """Opens what the CLI workspace (``axonml load``) remembers and the newest training log."""
        from ..cli.workspace import _ws_load
        ws = _ws_load()
        if ws.get("model") and self.model_view.model is None and os.path.exists(ws["model"]["path"]):
            self.load_model(ws["model"]["path"])
        if ws.get("dataset") and self.data_view.dataset is None and os.path.exists(ws["dataset"]["path"]):
            self.load_dataset(ws["dataset"]["path"])
        if self.training_view.session is None:
            log = find_training_log(self.cwd)
            if log:
                self.watch_training(log)
        self.go_to_tab(Tab.MODEL)

    def tick(self) -> bool:
        """Periodic work between key polls; True when the screen needs a redraw."""
        dirty = False
        if self.training_view.tick():
            self.graphs_view.set_session(self.training_view.session)
            dirty = True
        if self.status and time.monotonic() - self.status.at > self.STATUS_SECONDS:
            self.status, dirty = None, True
        return dirty

    # ------------------------------------------------------------------ keys
    def handle_key(self, key: str) -> None:
        if self.show_help:              # any key closes the overlay
            self.show_help = False
            return
        if key == "q":
            return self.quit()
        if key == "?":
            return self.toggle_help()
        if key == K.TAB:
            return self.next_tab()
        if key == K.BACKTAB:
            return self.prev_tab()
        if key in "123456" and len(key) == 1:
            return self.go_to_tab(Tab.all()[int(key) - 1])
        getattr(self, "_keys_" + self.active_tab.value.lower())(key)

    def _keys_model(self, key: str) -> None:
        v = self.model_view
        if key in (K.UP, "k"): v.select_prev()
        elif key in (K.DOWN, "j"): v.select_next()
        elif key == K.PAGE_UP: v.page(-10)
        elif key == K.PAGE_DOWN: v.page(10)
        elif key in (K.ENTER, "d"): v.toggle_details()

    def _keys_data(self, key: str) -> None:
        v = self.data_view
        if key in (K.UP, "k"): v.select_prev()
        elif key in (K.DOWN, "j"): v.select_next()
        elif key in (K.LEFT, "h"): v.prev_panel()
        elif key in (K.RIGHT, "l"): v.next_panel()

    def _keys_training(self, key: str) -> None:
        v = self.training_view
        if key in (K.UP, "k"): v.scroll_up()
        elif key in (K.DOWN, "j"): v.scroll_down()
        elif key == "d": v.toggle_details()
        elif key == "p":
            v.toggle_pause()
            self.set_status("paused: the log is no longer followed" if v.paused else "following the log again", StatusLevel.WARNING if v.paused else StatusLevel.INFO)
        elif key == "r":
            if not v.log_path:
                log = find_training_log(self.cwd)
                if log:
                    self.watch_training(log)
                else:
                    self.set_status("no training log found", StatusLevel.WARNING)
            elif v.refresh():
                self.graphs_view.set_session(v.session)
                self.set_status("training log re-read", StatusLevel.INFO)
            else:
                self.set_status(v.error or "training log unreadable", StatusLevel.ERROR)

    def _keys_graphs(self, key: str) -> None:
        v = self.graphs_view
        if key in (K.LEFT, "h"): v.prev_chart()
        elif key in (K.RIGHT, "l"): v.next_chart()
        elif key == "z": v.toggle_zoom()

    def _keys_files(self, key: str) -> None:
        v = self.files_view
        if key in (K.UP, "k"): v.select_prev()
        elif key in (K.DOWN, "j"): v.select_next()
        elif key == K.PAGE_UP: v.page(-10)
        elif key == K.PAGE_DOWN: v.page(10)
        elif key == K.ENTER:
            path = v.open_selected()
            if path:
                self.open_path(path)
        elif key in (K.RIGHT, "l"): v.enter_selected()
        elif key in (K.BACKSPACE, "u", "h", K.LEFT): v.go_up()
        elif key == "~": v.go_home()
        elif key == ".":
            v.toggle_hidden()
            self.set_status("dot files shown" if v.show_hidden else "dot files hidden")
        elif key == "o":
            if v.entries and v.entries[v.selected].file_type is FileType.DIRECTORY:
                self.load_dataset(v.entries[v.selected].path)
        elif key == "r":
            v.reload()

    def _keys_help(self, key: str) -> None:
        pass

    def open_path(self, path: str) -> None:
        """Routes a file to the view that shows it, by name."""
        low = path.lower()
        if os.path.basename(low) in _LOG_NAMES:
            self.watch_training(path)
        elif low.endswith(_MODEL_EXT):
            self.load_model(path)
        elif low.endswith(_DATA_EXT):
            self.load_dataset(path)
        else:
            self.set_status(os.path.basename(path) + ": previewed only (not a model, dataset or training log)")

    # ------------------------------------------------------------------ drawing
    def _header(self) -> Text:
        t = Text.assemble((" AxonML ", T.tab_active()), " ")
        for tab in Tab.all():
            t.append(f" {tab.key()}:{tab.value} ", style=T.tab_active() if tab is self.active_tab else T.tab_inactive())
        return t

    def _footer(self) -> Text:
        if self.status:
            return Text(" " + self.status.text, style=T.level(self.status.level.value))
        hints = {Tab.MODEL: "j/k layer   d details", Tab.DATA: "j/k row   h/l panel", Tab.TRAINING: "p pause   r re-read   d details",
                 Tab.GRAPHS: "h/l chart   z zoom", Tab.FILES: "Enter open   l enter   u parent   . hidden   o folder as dataset", Tab.HELP: ""}
        return Text(" q quit   ? help   Tab / 1-5 views   " + hints[self.active_tab], style=T.muted())

    def render(self):
        view = self.help_view if self.show_help else getattr(self, self.active_tab.value.lower() + "_view")
        title = "Help" if self.show_help else self.active_tab.value
        return Group(self._header(), Panel(view.render(), title=title, border_style=T.border()), self._footer())

    def frame(self, width: int = 120) -> str:
        """The current screen as plain text."""
        with open(os.devnull, "w") as sink:
            con = Console(width=width, record=True, file=sink, force_terminal=False, color_system=None)
            con.print(self.render())
            return con.export_text()

    def run_once(self, width: int = 120) -> str:
        """Every view rendered once, in tab order."""
        keep = self.active_tab
        out = []
        for tab in Tab.all():
            self.active_tab = tab
            out.append(self.frame(width))
        self.active_tab = keep
        return "\n".join(out)

    def run(self, poll_seconds: float = 0.1) -> None:
        """Interactive loop on a terminal (cbreak mode, alternate screen); one frame when stdin is not a TTY."""
        con = Console()
        if not sys.stdin.isatty():
            con.print(self.render())
            return
        import termios
        import tty
        from rich.live import Live
        fd = sys.stdin.fileno()
        old = termios.tcgetattr(fd)
        try:
            tty.setcbreak(fd)
            with Live(self.render(), console=con, screen=True, auto_refresh=False) as live:
                while not self.should_quit:
                    dirty = False
                    for key in K.read_keys(fd, poll_seconds):
                        self.handle_key(key)
                        dirty = True
                    dirty |= self.tick()
                    if dirty:
                        live.update(self.render(), refresh=True)
        finally:
            termios.tcsetattr(fd, termios.TCSADRAIN, old)


def run(model_path: str | None = None, data_path: str | None = None, watch: str | None = None, cwd: str = ".") -> None:
    """Entry point of ``axonml tui`` (crates/axonml-tui/src/lib.rs ``run``)."""
    app = build_app(model_path, data_path, watch, cwd)
    app.run()


def build_app(model_path: str | None = None, data_path: str | None = None, watch: str | None = None, cwd: str = ".") -> App:
    app = App(cwd)
    if model_path:
        app.load_model(model_path)
    if data_path:
        app.load_dataset(data_path)
    if watch:
        app.watch_training(watch)
    app.load_workspace()
    if watch:
        app.go_to_tab(Tab.TRAINING)
    return app
