"""Graphs view: loss, accuracy and learning-rate curves of the watched run, drawn with braille dots.

Parity: crates/axonml-tui/src/views/graphs.rs (``ChartType{Loss, Accuracy, LearningRate}``,
``DataSeries``, ``GraphsView`` with train / validation series, axis bounds, ``next_chart`` /
``prev_chart`` and ``toggle_zoom``).  The reference plots demo curves through ratatui's ``Chart``
widget; here the series come from the Training view's session and the chart is rasterised on a
braille canvas (2 x 4 dots per character cell)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from rich.console import Group
from rich.panel import Panel
from rich.text import Text

from ..theme import AxonmlTheme as T

# dot bit of (column, row) inside one braille cell
_DOT = ((0x01, 0x02, 0x04, 0x40), (0x08, 0x10, 0x20, 0x80))


class ChartType(Enum):
    LOSS = "Loss"
    ACCURACY = "Accuracy"
    LEARNING_RATE = "Learning Rate"


@dataclass
class DataSeries:
    name: str
    data: list = field(default_factory=list)      # (x, y) points
    colour: str = ""


class BrailleCanvas:
    """A grid of ``width`` x ``height`` character cells addressed in dots (2 per cell across, 4 down)."""

    def __init__(self, width: int, height: int):
        self.w, self.h = width, height
        self.bits = [[0] * width for _ in range(height)]
        self.colour = [[""] * width for _ in range(height)]

    def set(self, px: int, py: int, colour: str) -> None:
        if 0 <= px < 2 * self.w and 0 <= py < 4 * self.h:
            cx, cy = px // 2, py // 4
            self.bits[cy][cx] |= _DOT[px % 2][py % 4]
            self.colour[cy][cx] = colour

    def line(self, x0: int, y0: int, x1: int, y1: int, colour: str) -> None:
        dx, dy = abs(x1 - x0), -abs(y1 - y0)
        sx, sy = (1 if x0 < x1 else -1), (1 if y0 < y1 else -1)
        err = dx + dy
        while True:
            self.set(x0, y0, colour)
            if x0 == x1 and y0 == y1:
                return
            e2 = 2 * err
            if e2 >= dy:
                err += dy
                x0 += sx
            if e2 <= dx:
                err += dx
                y0 += sy

    def rows(self) -> list[Text]:
        out = []
        for bits, cols in zip(self.bits, self.colour):
            t = Text()
            for b, c in zip(bits, cols):
                t.append(chr(0x2800 + b) if b else " ", style=c or None)
            out.append(t)
        return out


def plot(series: list, x_bounds, y_bounds, width: int = 90, height: int = 16) -> list[Text]:
    """Chart rows (y-axis labels, canvas, x-axis line) of the series within the bounds."""
    (x0, x1), (y0, y1) = x_bounds, y_bounds
    if x1 <= x0:
        x1 = x0 + 1
    if y1 <= y0:
        y1 = y0 + 1
    cv = BrailleCanvas(width, height)
    pw, ph = 2 * width - 1, 4 * height - 1
    for s in series:
        prev = None
        for x, y in s.data:
            if x < x0 or x > x1:
                prev = None
                continue
            px = round((x - x0) / (x1 - x0) * pw)
            py = ph - round((min(max(y, y0), y1) - y0) / (y1 - y0) * ph)
            if prev is None:
                cv.set(px, py, s.colour)
            else:
                cv.line(prev[0], prev[1], px, py, s.colour)
            prev = (px, py)
    fmt = (lambda v: f"{v:9.2e}") if max(abs(y0), abs(y1)) < 1e-2 else (lambda v: f"{v:9.3f}")
    rows = []
    for i, r in enumerate(cv.rows()):
        label = fmt(y1) if i == 0 else fmt(y0) if i == height - 1 else fmt((y0 + y1) / 2) if i == height // 2 else " " * 9
        rows.append(Text.assemble((label, T.muted()), (" ┤" if label.strip() else " │", T.border()), r))
    rows.append(Text(" " * 10 + "└" + "─" * width, style=T.border()))
    left, right = f"{x0:g}", f"{x1:g}"
    rows.append(Text(" " * 11 + left + " " * max(width - len(left) - len(right), 1) + right, style=T.muted()))
    return rows


class GraphsView:
    def __init__(self):
        self.train_loss: list = []
        self.val_loss: list = []
        self.train_acc: list = []
        self.val_acc: list = []
        self.learning_rate: list = []
        self.active_chart = ChartType.LOSS
        self.zoomed = False
        self.x_bounds = [0.0, 1.0]
        self.loss_bounds = [0.0, 1.0]
        self.acc_bounds = [0.0, 100.0]

    def set_session(self, session) -> None:
        """Takes the curves of a ``TrainingSession`` (or clears them when ``None``)."""
        hist = session.metrics_history if session is not None else []
        pick = lambda attr: [(float(m.epoch), float(getattr(m, attr))) for m in hist if getattr(m, attr) is not None]
        self.train_loss, self.val_loss = pick("train_loss"), pick("val_loss")
        self.train_acc, self.val_acc = pick("train_acc"), pick("val_acc")
        self.learning_rate = pick("learning_rate")
        if hist:
            self.x_bounds = [float(hist[0].epoch), float(max(hist[-1].epoch, hist[0].epoch + 1))]
        ys = [y for _, y in self.train_loss + self.val_loss]
        if ys:
            self.loss_bounds = [0.0 if min(ys) >= 0 else min(ys), max(ys) * 1.05 or 1.0]
        accs = [y for _, y in self.train_acc + self.val_acc]
        self.acc_bounds = [0.0, 100.0 if accs and max(accs) > 1.0 else 1.0]

    def next_chart(self) -> None:
        order = list(ChartType)
        self.active_chart = order[(order.index(self.active_chart) + 1) % len(order)]

    def prev_chart(self) -> None:
        order = list(ChartType)
        self.active_chart = order[(order.index(self.active_chart) - 1) % len(order)]

    def toggle_zoom(self) -> None:
        """Zoomed in, the chart shows the second half of the run with the y-axis fitted to it."""
        self.zoomed = not self.zoomed

    def series(self) -> list:
        if self.active_chart is ChartType.LOSS:
            return [DataSeries("train loss", self.train_loss, T.series(0)), DataSeries("validation loss", self.val_loss, T.series(1))]
        if self.active_chart is ChartType.ACCURACY:
            return [DataSeries("train accuracy", self.train_acc, T.series(3)), DataSeries("validation accuracy", self.val_acc, T.series(2))]
        return [DataSeries("learning rate", self.learning_rate, T.series(4))]

    def bounds(self):
        ss = [s for s in self.series() if s.data]
        xb = list(self.x_bounds)
        if self.zoomed:
            xb[0] = xb[0] + (xb[1] - xb[0]) / 2
        ys = [y for s in ss for x, y in s.data if xb[0] <= x <= xb[1]]
        if self.active_chart is ChartType.LOSS and not self.zoomed:
            yb = list(self.loss_bounds)
        elif self.active_chart is ChartType.ACCURACY and not self.zoomed:
            yb = list(self.acc_bounds)
        elif ys:
            pad = (max(ys) - min(ys)) * 0.05 or abs(max(ys)) * 0.05 or 1.0
            yb = [min(ys) - pad, max(ys) + pad]
        else:
            yb = [0.0, 1.0]
        return xb, yb

    def render(self, width: int = 90, height: int = 16):
        tabs = Text()
        for c in ChartType:
            tabs.append(f" {c.value} ", style=T.tab_active() if c is self.active_chart else T.tab_inactive())
        if self.zoomed:
            tabs.append("  zoom: second half", style=T.warning())
        ss = [s for s in self.series() if s.data]
        if not ss:
            return Group(tabs, Panel(Text("nothing to plot: the watched run has no " + self.active_chart.value.lower() + " values yet",
                                          style=T.muted()), title=self.active_chart.value, border_style=T.border()))
        xb, yb = self.bounds()
        legend = Text()
        for s in ss:
            legend.append("━━ ", style=s.colour)
            legend.append(f"{s.name} (last {s.data[-1][1]:.4g})   ", style=T.muted())
        return Group(tabs, Panel(Group(*plot(ss, xb, yb, width, height), legend), title=f"{self.active_chart.value} by epoch",
                                 border_style=T.border_focused()))
