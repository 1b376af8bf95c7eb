"""Model view: the layers of a model file with their kind, shapes and parameter counts.

Parity: crates/axonml-tui/src/views/model.rs (``LayerInfo``, ``ModelInfo``, ``ModelView`` with
``load_model``, ``select_prev`` / ``select_next``, ``toggle_details``, a layer list beside a
details panel and a summary line).  The reference infers layers from the entries of a state
dictionary; so does this view, for every format the registry reads (.axonml, safetensors, GGUF,
ONNX)."""
from __future__ import annotations

import os
from dataclasses import dataclass, field

from rich.console import Group
from rich.panel import Panel
from rich.table import Table
from rich.text import Text

from ..theme import AxonmlTheme as T

_DTYPE_BYTES = {"float32": 4, "float": 4, "f32": 4, "float16": 2, "f16": 2, "bfloat16": 2, "bf16": 2, "float64": 8,
                "int8": 1, "uint8": 1, "int32": 4, "int64": 8, "bool": 1}
_EMBED_HINTS = ("embed", "wte", "wpe", "tok_", "token", "position")


@dataclass
class LayerInfo:
    name: str
    layer_type: str
    input_shape: str
    output_shape: str
    params: int
    trainable: bool = True
    tensors: list = field(default_factory=list)      # (suffix, shape, dtype)
    bytes: int = 0


@dataclass
class ModelInfo:
    name: str
    layers: list
    total_params: int
    trainable_params: int
    file_size: int
    format: str
    path: str = ""


def format_count(n: int) -> str:
    for unit, div in (("B", 1e9), ("M", 1e6), ("K", 1e3)):
        if n >= div:
            return f"{n / div:.2f}{unit}"
    return str(n)


def format_size(n: int) -> str:
    for unit, div in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if n >= div:
            return f"{n / div:.1f} {unit}"
    return f"{n} B"


def classify_layer(stem: str, tensors: dict) -> tuple[str, str, str]:
    """(kind, input shape, output shape) of the layer whose tensors are ``{suffix: shape}``."""
    w = tensors.get("weight")
    if w is None:
        w = next((s for k, s in tensors.items() if k not in ("bias", "running_mean", "running_var", "num_batches_tracked")), None)
    if w is None:
        return "Bias", "-", "-"
    low = stem.lower()
    if len(w) == 2:
        if any(h in low for h in _EMBED_HINTS):
            return "Embedding", "[*]", f"[*, {w[1]}]"
        return "Linear", f"[*, {w[1]}]", f"[*, {w[0]}]"
    if len(w) == 4:
        return "Conv2d", f"[N, {w[1]}, H, W]", f"[N, {w[0]}, H', W']  k={w[2]}x{w[3]}"
    if len(w) == 3:
        return "Conv1d", f"[N, {w[1]}, L]", f"[N, {w[0]}, L']  k={w[2]}"
    if len(w) == 1:
        if "running_mean" in tensors:
            kind = "BatchNorm"
        elif "bias" not in tensors:
            kind = "RMSNorm"
        else:
            kind = "LayerNorm"
        return kind, f"[*, {w[0]}]", f"[*, {w[0]}]"
    return "Tensor", "-", str(list(w))


def model_info(path: str) -> ModelInfo:
    from ...cli.workspace import model_summary
    s = model_summary(path)
    groups: dict[str, list] = {}
    for e in s["entries"]:
        stem, _, suffix = e["name"].rpartition(".")
        if not stem:
            stem, suffix = e["name"], "weight"
        groups.setdefault(stem, []).append((suffix, list(e["shape"]), e["dtype"], e["numel"]))
    layers = []
    for stem, ts in groups.items():
        kind, i, o = classify_layer(stem, {sfx: shp for sfx, shp, _, _ in ts})
        nbytes = sum(n * _DTYPE_BYTES.get(str(dt).lower(), 4) for _, _, dt, n in ts)
        frozen = all(sfx in ("running_mean", "running_var", "num_batches_tracked") for sfx, _, _, _ in ts)
        params = sum(n for sfx, _, _, n in ts if sfx not in ("running_mean", "running_var", "num_batches_tracked"))
        layers.append(LayerInfo(stem, kind, i, o, params, not frozen, [(sfx, shp, dt) for sfx, shp, dt, _ in ts], nbytes))
    total = sum(l.params for l in layers)
    return ModelInfo(os.path.basename(path), layers, total, sum(l.params for l in layers if l.trainable),
                     s["file_bytes"], s["format"], s["path"])


class ModelView:
    VISIBLE = 22

    def __init__(self):
        self.model: ModelInfo | None = None
        self.selected_layer = 0
        self.show_details = True
        self.error = ""

    def load_model(self, path: str) -> None:
        """Raises on an unreadable file; the previous model stays loaded then."""
        self.model = model_info(path)
        self.selected_layer, self.error = 0, ""

    def select_prev(self) -> None:
        if self.selected_layer > 0:
            self.selected_layer -= 1

    def select_next(self) -> None:
        if self.model and self.selected_layer < len(self.model.layers) - 1:
            self.selected_layer += 1

    def page(self, delta: int) -> None:
        if self.model:
            self.selected_layer = min(max(self.selected_layer + delta, 0), len(self.model.layers) - 1)

    def toggle_details(self) -> None:
        self.show_details = not self.show_details

    # ------------------------------------------------------------------ drawing
    def _layer_table(self) -> Table:
        m = self.model
        tb = Table(expand=True, box=None, pad_edge=False)
        tb.add_column("#", justify="right", style=T.muted(), width=4)
        tb.add_column("layer", ratio=3, no_wrap=True)
        tb.add_column("type", min_width=10, no_wrap=True)
        tb.add_column("output", ratio=2, no_wrap=True)
        tb.add_column("params", justify="right", ratio=1)
        lo = max(0, min(self.selected_layer - self.VISIBLE // 2, len(m.layers) - self.VISIBLE))
        for i, l in enumerate(m.layers[lo:lo + self.VISIBLE], start=lo):
            style = T.selected() if i == self.selected_layer else None
            tb.add_row(str(i), l.name, Text(l.layer_type, style=None if style else T.layer(l.layer_type)), l.output_shape,
                       format_count(l.params), style=style)
        return tb

    def _details(self) -> Group:
        l = self.model.layers[self.selected_layer]
        share = 100.0 * l.params / max(self.model.total_params, 1)
        rows = [("name", l.name), ("type", l.layer_type), ("input", l.input_shape), ("output", l.output_shape),
                ("parameters", f"{l.params:,}  ({share:.1f} % of the model)"), ("memory", format_size(l.bytes)),
                ("trainable", "yes" if l.trainable else "no (buffers)")]
        tb = Table(box=None, show_header=False, pad_edge=False)
        tb.add_column(style=T.muted()); tb.add_column()
        for k, v in rows:
            tb.add_row(k, v)
        tt = Table(box=None, pad_edge=False, title="tensors", title_style=T.header(), title_justify="left")
        tt.add_column("name"); tt.add_column("shape"); tt.add_column("dtype", style=T.muted())
        for sfx, shp, dt in l.tensors:
            tt.add_row(sfx, "x".join(map(str, shp)) or "scalar", str(dt))
        return Group(tb, Text(""), tt)

    def render(self):
        if self.model is None:
            msg = self.error or "no model loaded: open one from the Files view (5) or start with --model <file>"
            return Text(msg, style=T.error() if self.error else T.muted())
        m = self.model
        summary = Text.assemble((m.name, T.title()), "  ", (m.format, T.accent()), "  ", (f"{len(m.layers)} layers", T.muted()), "  ",
                                (f"{m.total_params:,} parameters", T.metric_value()), "  ",
                                (f"{m.trainable_params:,} trainable", T.muted()), "  ", (format_size(m.file_size), T.muted()))
        left = Panel(self._layer_table(), title=f"Layers ({self.selected_layer + 1}/{len(m.layers)})", border_style=T.border_focused())
        if not self.show_details:
            return Group(summary, left)
        grid = Table.grid(expand=True)
        grid.add_column(ratio=3); grid.add_column(ratio=2)
        grid.add_row(left, Panel(self._details(), title="Details", border_style=T.border()))
        return Group(summary, grid)
