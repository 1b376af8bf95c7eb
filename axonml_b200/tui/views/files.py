"""Files view: a directory tree with expandable folders, a preview pane and typed entries.

Parity: crates/axonml-tui/src/views/files.rs (``FileType{Directory, Model, Dataset, Config,
Other}`` from the extension, ``FileEntry{name, path, file_type, size, is_expanded, depth}``,
``FilesView`` with ``select_prev`` / ``select_next``, ``toggle_or_open``, ``open_selected``,
``go_parent`` / ``go_up``, ``go_home``, ``toggle_hidden``, a filter and a preview of the selected
entry).  The reference lists demo entries; this view reads the file system."""
from __future__ import annotations

import os
from dataclasses import dataclass
from enum import Enum
from itertools import islice

from rich.panel import Panel
from rich.table import Table
from rich.text import Text

from ..theme import AxonmlTheme as T
from .model import format_size

_MODEL_EXT = {"axonml", "onnx", "pt", "pth", "safetensors", "st", "gguf", "h5", "keras", "bin"}
_DATA_EXT = {"npz", "npy", "csv", "tsv", "parquet", "arrow", "tfrecord", "idx", "idx1-ubyte", "idx3-ubyte"}
_CONFIG_EXT = {"toml", "yaml", "yml", "json", "jsonl"}
_TEXT_EXT = _CONFIG_EXT | {"txt", "md", "py", "log", "csv", "tsv", "cfg", "ini", "sh"}


class FileType(Enum):
    DIRECTORY = "Directory"
    MODEL = "Model"
    DATASET = "Dataset"
    CONFIG = "Config"
    OTHER = "Other"

    def icon(self) -> str:
        return {"Directory": "▸", "Model": "◆", "Dataset": "▦", "Config": "⚙", "Other": "·"}[self.value]

    def style(self) -> str:
        return {"Directory": T.header(), "Model": T.success(), "Dataset": T.info(), "Config": T.accent(), "Other": ""}[self.value]

    @classmethod
    def from_extension(cls, ext: str) -> "FileType":
        e = ext.lower().lstrip(".")
        if e in _MODEL_EXT:
            return cls.MODEL
        if e in _DATA_EXT:
            return cls.DATASET
        if e in _CONFIG_EXT:
            return cls.CONFIG
        return cls.OTHER


@dataclass
class FileEntry:
    name: str
    path: str
    file_type: FileType
    depth: int = 0
    size: int | None = None
    is_expanded: bool = False


class FilesView:
    VISIBLE = 24
    MAX_CHILDREN = 500

    def __init__(self, cwd: str = "."):
        self.current_dir = os.path.abspath(cwd)
        self.entries: list[FileEntry] = []
        self.selected = 0
        self.show_hidden = False
        self.filter: str | None = None
        self.preview: str | None = None
        self._expanded: set[str] = set()
        self.reload()

    # ------------------------------------------------------------------ listing
    def _children(self, directory: str, depth: int) -> list[FileEntry]:
        try:
            names = sorted(os.listdir(directory), key=str.lower)
        except OSError:
            return []
        dirs, files = [], []
        for n in names[:self.MAX_CHILDREN]:
            if n.startswith(".") and not self.show_hidden:
                continue
            p = os.path.join(directory, n)
            if os.path.isdir(p):
                dirs.append(FileEntry(n, p, FileType.DIRECTORY, depth, None, p in self._expanded))
            else:
                if self.filter and self.filter.lower() not in n.lower():
                    continue
                try:
                    size = os.path.getsize(p)
                except OSError:
                    size = None
                files.append(FileEntry(n, p, FileType.from_extension(os.path.splitext(n)[1]), depth, size))
        out = []
        for d in dirs:
            out.append(d)
            if d.is_expanded:
                out += self._children(d.path, depth + 1)
        return out + files

    def reload(self) -> None:
        keep = self.entries[self.selected].path if self.entries and self.selected < len(self.entries) else None
        self.entries = self._children(self.current_dir, 0)
        self.selected = next((i for i, e in enumerate(self.entries) if e.path == keep), min(self.selected, max(len(self.entries) - 1, 0)))
        self.update_preview()

    # ------------------------------------------------------------------ movement
    def select_prev(self) -> None:
        if self.selected > 0:
            self.selected -= 1
            self.update_preview()

    def select_next(self) -> None:
        if self.selected < len(self.entries) - 1:
            self.selected += 1
            self.update_preview()

    def page(self, delta: int) -> None:
        if self.entries:
            self.selected = min(max(self.selected + delta, 0), len(self.entries) - 1)
            self.update_preview()

    def toggle_or_open(self) -> None:
        """Expands or collapses the selected directory in place."""
        if not self.entries:
            return
        e = self.entries[self.selected]
        if e.file_type is FileType.DIRECTORY:
            (self._expanded.discard if e.path in self._expanded else self._expanded.add)(e.path)
            self.reload()

    def open_selected(self) -> str | None:
        """Path of the selected file; a directory is toggled instead and ``None`` returned."""
        if not self.entries:
            return None
        e = self.entries[self.selected]
        if e.file_type is FileType.DIRECTORY:
            self.toggle_or_open()
            return None
        return e.path

    def enter_selected(self) -> None:
        """Makes the selected directory the root of the listing."""
        if self.entries and self.entries[self.selected].file_type is FileType.DIRECTORY:
            self.current_dir, self.selected = self.entries[self.selected].path, 0
            self.reload()

    def go_parent(self) -> None:
        parent = os.path.dirname(self.current_dir)
        if parent and parent != self.current_dir:
            child = self.current_dir
            self.current_dir = parent
            self.entries, self.selected = [], 0
            self.reload()
            self.selected = next((i for i, e in enumerate(self.entries) if e.path == child), 0)
            self.update_preview()

    go_up = go_parent

    def go_home(self) -> None:
        self.current_dir, self.entries, self.selected = os.path.expanduser("~"), [], 0
        self.reload()

    def toggle_hidden(self) -> None:
        self.show_hidden = not self.show_hidden
        self.reload()

    def set_filter(self, pattern: str | None) -> None:
        self.filter = pattern or None
        self.reload()

    # ------------------------------------------------------------------ preview
    def update_preview(self) -> None:
        if not self.entries:
            self.preview = None
            return
        e = self.entries[self.selected]
        lines = [f"Path: {e.path}", f"Type: {e.file_type.value}", f"Size: {format_size(e.size) if e.size is not None else '-'}"]
        if e.file_type is FileType.DIRECTORY:
            try:
                kids = os.listdir(e.path)
                lines.append(f"Entries: {len(kids)}")
            except OSError as err:
                lines.append(f"unreadable: {err.strerror}")
        elif os.path.splitext(e.name)[1].lower().lstrip(".") in _TEXT_EXT and (e.size or 0) > 0:
            try:
                with open(e.path, errors="replace") as f:
                    head = [l.rstrip("\n")[:100] for l in islice(f, 12)]
            except OSError:
                head = []
            lines += ["", *head]
        elif e.file_type is FileType.MODEL:
            lines += ["", "Enter: open in the Model view"]
        elif e.file_type is FileType.DATASET:
            lines += ["", "Enter: open in the Data view"]
        self.preview = "\n".join(lines)

    # ------------------------------------------------------------------ drawing
    def render(self):
        tb = Table(expand=True, box=None, pad_edge=False, show_header=False)
        tb.add_column(ratio=5, no_wrap=True); tb.add_column(justify="right", ratio=1, no_wrap=True)
        lo = max(0, min(self.selected - self.VISIBLE // 2, len(self.entries) - self.VISIBLE))
        for i, e in enumerate(self.entries[lo:lo + self.VISIBLE], start=lo):
            icon = ("▾" if e.is_expanded else "▸") if e.file_type is FileType.DIRECTORY else e.file_type.icon()
            name = Text("  " * e.depth + icon + " " + e.name + ("/" if e.file_type is FileType.DIRECTORY else ""),
                        style=None if i == self.selected else (e.file_type.style() or None))
            tb.add_row(name, "" if e.size is None else format_size(e.size), style=T.selected() if i == self.selected else None)
        if not self.entries:
            tb.add_row(Text("(empty)", style=T.muted()), "")
        title = self.current_dir + ("  [hidden shown]" if self.show_hidden else "") + (f"  [filter: {self.filter}]" if self.filter else "")
        grid = Table.grid(expand=True)
        grid.add_column(ratio=3); grid.add_column(ratio=2)
        grid.add_row(Panel(tb, title=title, border_style=T.border_focused()),
                     Panel(Text(self.preview or "", overflow="ellipsis", no_wrap=True), title="Preview", border_style=T.border()))
        return grid
