"""Data view: class distribution, features and splits of a dataset on disk.

Parity: crates/axonml-tui/src/views/data.rs (``ClassInfo``, ``SplitInfo``, ``FeatureInfo``,
``DatasetInfo``; ``DataView`` with a class list, a feature table, a split bar, ``select_prev`` /
``select_next`` and ``prev_panel`` / ``next_panel``).  The reference view shows built-in demo data;
this one analyses the dataset it is given (CSV / TSV tables, image folders, IDX files, text)."""
from __future__ import annotations

import os
from dataclasses import dataclass, field

from rich.console import Group
from rich.panel import Panel
from rich.table import Table
from rich.text import Text

from ..theme import AxonmlTheme as T
from .model import format_size

PANELS = ["Classes", "Features"]
_SPLIT_DIRS = {"train": "train", "training": "train", "val": "validation", "valid": "validation", "validation": "validation",
               "test": "test", "testing": "test"}


@dataclass
class ClassInfo:
    name: str
    count: int
    percentage: float


@dataclass
class SplitInfo:
    name: str
    samples: int
    percentage: float


@dataclass
class FeatureInfo:
    name: str
    dtype: str
    shape: str
    min: float | None = None
    max: float | None = None
    mean: float | None = None
    missing: int = 0


@dataclass
class DatasetInfo:
    name: str
    total_samples: int
    num_classes: int
    feature_dim: str
    classes: list = field(default_factory=list)
    splits: list = field(default_factory=list)
    features: list = field(default_factory=list)
    file_path: str = ""
    file_size: int = 0
    kind: str = ""
    task: str = ""
    imbalance_ratio: float | None = None
    recommendations: dict = field(default_factory=dict)


def _count_files(path: str) -> int:
    return sum(len(fs) for _, _, fs in os.walk(path))


def _splits(path: str, total: int, val_split: float) -> list:
    """Split sizes from train/ val/ test/ sub-directories when the dataset has them, else the split
    the recommended validation fraction gives."""
    found = {}
    if os.path.isdir(path):
        for d in sorted(os.listdir(path)):
            name = _SPLIT_DIRS.get(d.lower())
            if name and os.path.isdir(os.path.join(path, d)):
                found[name] = found.get(name, 0) + _count_files(os.path.join(path, d))
    if not found:
        n_val = int(round(total * val_split))
        found = {"train": total - n_val, "validation": n_val}
    tot = sum(found.values()) or 1
    return [SplitInfo(k, v, 100.0 * v / tot) for k, v in found.items()]


def dataset_info(path: str, max_samples: int = 10_000) -> DatasetInfo:
    from ...data.analysis import analyze_dataset
    a = analyze_dataset(path, max_samples=max_samples)
    total = int(a.get("num_samples") or 0)
    cc = a.get("class_counts") or {}
    ctot = sum(cc.values()) or 1
    classes = [ClassInfo(str(k), int(v), 100.0 * v / ctot) for k, v in sorted(cc.items(), key=lambda kv: (-kv[1], str(kv[0])))]
    feats = []
    for c in a.get("columns") or []:
        feats.append(FeatureInfo(c["name"], c["dtype"], "[1]", c.get("min"), c.get("max"), c.get("mean"), c.get("missing", 0)))
    if a.get("image_shape"):
        shp = a["image_shape"]
        feats.append(FeatureInfo("image", "uint8", "[" + ", ".join(map(str, shp)) + "]", 0.0, 255.0, None))
        feats.append(FeatureInfo("label", "int64", "[1]", 0.0, float(max(len(cc) - 1, 0)), None))
        dim = "x".join(map(str, shp))
    elif a.get("num_features"):
        dim = str(a["num_features"])
    else:
        dim = "-"
    rec = a.get("recommendations") or {}
    return DatasetInfo(os.path.basename(os.path.normpath(path)), total, len(cc), dim, classes,
                       _splits(path, total, float(rec.get("val_split", 0.2))), feats, a["path"], int(a.get("size_bytes") or 0),
                       a.get("dataset_type", ""), a.get("task", ""), a.get("imbalance_ratio"), rec)


class DataView:
    VISIBLE = 18

    def __init__(self):
        self.dataset: DatasetInfo | None = None
        self.selected_class = 0
        self.selected_feature = 0
        self.active_panel = 0
        self.error = ""

    def load_dataset(self, path: str) -> None:
        self.dataset = dataset_info(path)
        self.selected_class = self.selected_feature = 0
        self.error = ""

    def _len(self) -> int:
        if self.dataset is None:
            return 0
        return len(self.dataset.classes) if self.active_panel == 0 else len(self.dataset.features)

    def select_prev(self) -> None:
        if self.active_panel == 0:
            self.selected_class = max(self.selected_class - 1, 0)
        else:
            self.selected_feature = max(self.selected_feature - 1, 0)

    def select_next(self) -> None:
        hi = max(self._len() - 1, 0)
        if self.active_panel == 0:
            self.selected_class = min(self.selected_class + 1, hi)
        else:
            self.selected_feature = min(self.selected_feature + 1, hi)

    def next_panel(self) -> None:
        self.active_panel = (self.active_panel + 1) % len(PANELS)

    def prev_panel(self) -> None:
        self.active_panel = (self.active_panel - 1) % len(PANELS)

    switch_panel = next_panel

    # ------------------------------------------------------------------ drawing
    def _classes(self) -> Table:
        d = self.dataset
        tb = Table(expand=True, box=None, pad_edge=False)
        tb.add_column("class", ratio=2, no_wrap=True); tb.add_column("count", justify="right", ratio=1)
        tb.add_column("share", justify="right", ratio=1); tb.add_column("", ratio=4, no_wrap=True)
        top = max((c.percentage for c in d.classes), default=1.0) or 1.0
        lo = max(0, min(self.selected_class - self.VISIBLE // 2, len(d.classes) - self.VISIBLE))
        for i, c in enumerate(d.classes[lo:lo + self.VISIBLE], start=lo):
            sel = self.active_panel == 0 and i == self.selected_class
            tb.add_row(c.name, f"{c.count:,}", f"{c.percentage:.1f}%", Text("█" * max(1, int(32 * c.percentage / top)), style=T.series(i)),
                       style=T.selected() if sel else None)
        if not d.classes:
            tb.add_row(Text("no class labels found" if d.task != "regression" else "regression target", style=T.muted()), "", "", "")
        return tb

    def _features(self) -> Table:
        d = self.dataset
        tb = Table(expand=True, box=None, pad_edge=False)
        for c, j in (("feature", "left"), ("dtype", "left"), ("shape", "left"), ("min", "right"), ("max", "right"), ("mean", "right"),
                     ("missing", "right")):
            tb.add_column(c, justify=j, no_wrap=True)
        f = lambda v: "-" if v is None else f"{v:.4g}"
        lo = max(0, min(self.selected_feature - self.VISIBLE // 2, len(d.features) - self.VISIBLE))
        for i, x in enumerate(d.features[lo:lo + self.VISIBLE], start=lo):
            sel = self.active_panel == 1 and i == self.selected_feature
            tb.add_row(x.name, x.dtype, x.shape, f(x.min), f(x.max), f(x.mean), str(x.missing), style=T.selected() if sel else None)
        if not d.features:
            tb.add_row(Text("no per-feature statistics for this dataset type", style=T.muted()), "", "", "", "", "", "")
        return tb

    def _split_bar(self, width: int = 72) -> Text:
        t = Text()
        for i, s in enumerate(self.dataset.splits):
            label = f" {s.name} {s.samples:,} ({s.percentage:.0f}%) "
            w = max(len(label), int(width * s.percentage / 100.0))
            t.append(label.center(w), style=f"bold #1e293b on {T.series(i)}")
        return t

    def render(self):
        if self.dataset is None:
            msg = self.error or "no dataset loaded: open one from the Files view (5) or start with --data <path>"
            return Text(msg, style=T.error() if self.error else T.muted())
        d = self.dataset
        head = Text.assemble((d.name, T.title()), "  ", (d.kind, T.accent()), "  ", (d.task or "", T.muted()), "  ",
                             (f"{d.total_samples:,} samples", T.metric_value()), "  ", (f"{d.num_classes} classes", T.muted()), "  ",
                             (f"features {d.feature_dim}", T.muted()), "  ", (format_size(d.file_size), T.muted()))
        if d.imbalance_ratio and d.imbalance_ratio > 3:
            head.append(f"  imbalance {d.imbalance_ratio:.1f}x", style=T.warning())
        grid = Table.grid(expand=True)
        grid.add_column(ratio=1); grid.add_column(ratio=1)
        grid.add_row(Panel(self._classes(), title="Classes", border_style=T.border_focused() if self.active_panel == 0 else T.border()),
                     Panel(self._features(), title="Features", border_style=T.border_focused() if self.active_panel == 1 else T.border()))
        rec = ", ".join(f"{k}={v}" for k, v in d.recommendations.items() if k != "notes")
        notes = [Text(n, style=T.warning()) for n in d.recommendations.get("notes", [])]
        return Group(head, grid, Panel(self._split_bar(), title="Splits", border_style=T.border()),
                     Text("recommended: " + rec, style=T.muted()), *notes)
