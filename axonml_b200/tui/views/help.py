"""Help view: the key map, global keys first and then one section per view.

Parity: crates/axonml-tui/src/views/help.rs (``HelpView`` listing the global, navigation and
per-view key bindings beside a short description of each view)."""
from __future__ import annotations

from rich.console import Group
from rich.panel import Panel
from rich.table import Table
from rich.text import Text

from ..theme import AxonmlTheme as T

SECTIONS = [
    ("Global", [("q / Ctrl-C", "quit"), ("?", "toggle this help over any view"), ("Tab / Shift-Tab", "next / previous view"),
                ("1 - 5", "Model, Data, Training, Graphs, Files"), ("6", "help view")]),
    ("Model", [("j k / arrows", "select a layer"), ("PgUp PgDn", "move ten layers"), ("Enter / d", "show or hide the details panel")]),
    ("Data", [("j k / arrows", "select a class or feature"), ("h l / arrows", "switch between the Classes and Features panels")]),
    ("Training", [("j k / arrows", "scroll the epoch table"), ("p", "pause or resume following the log"), ("r", "re-read the log now"),
                  ("d", "show or hide the run panel")]),
    ("Graphs", [("h l / arrows", "previous / next chart (loss, accuracy, learning rate)"), ("z", "zoom on the second half of the run")]),
    ("Files", [("j k / arrows", "select an entry"), ("Enter", "expand a folder; open a model, dataset or training log"),
               ("l / right", "make the selected folder the root"), ("Backspace / u / h", "parent folder"), ("~", "home folder"),
               (".", "show or hide dot files"), ("o", "open the selected folder as a dataset"), ("r", "re-read the folder")]),
]
VIEW_NOTES = [
    ("Model", "layers of a model file (.axonml, safetensors, GGUF, ONNX) with kinds, shapes and parameter counts"),
    ("Data", "class balance, per-feature statistics and splits of a dataset on disk"),
    ("Training", "progress, metrics and ETA of a run, followed live from its JSON-lines log"),
    ("Graphs", "loss, accuracy and learning-rate curves of the watched run"),
    ("Files", "folder tree with previews; the way to open things in the other views"),
]


class HelpView:
    def keys(self) -> list:
        """Flat (section, key, action) rows."""
        return [(s, k, a) for s, rows in SECTIONS for k, a in rows]

    def render(self):
        tb = Table(expand=True, box=None, pad_edge=False, show_header=False)
        tb.add_column(width=10, style=T.header()); tb.add_column(width=20, style=T.key()); tb.add_column(ratio=1)
        for section, rows in SECTIONS:
            for i, (k, a) in enumerate(rows):
                tb.add_row(section if i == 0 else "", k, a)
            tb.add_row("", "", "")
        notes = Table(expand=True, box=None, pad_edge=False, show_header=False)
        notes.add_column(width=10, style=T.header()); notes.add_column(ratio=1, style=T.muted())
        for v, n in VIEW_NOTES:
            notes.add_row(v, n)
        return Group(Panel(tb, title="Keys", border_style=T.border_focused()), Panel(notes, title="Views", border_style=T.border()),
                     Text("AxonML terminal interface", style=T.muted()))
