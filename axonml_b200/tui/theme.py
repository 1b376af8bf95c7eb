"""Colours and named styles of the terminal interface.

Parity: crates/axonml-tui/src/theme.rs (brand palette: teal primary, terracotta accent, cream /
dark-slate surfaces; semantic success / warning / error / info colours; style helpers ``header``,
``selected``, ``muted``, ``border``, ``border_focused``, ``tab_active`` ..., one colour per layer
type and per graph series).  Styles are ``rich`` style strings."""
from __future__ import annotations

TEAL = "#14b8a6"
TEAL_LIGHT = "#5eead4"
TERRACOTTA = "#c4a484"
CREAM = "#faf9f6"
DARK_SLATE = "#1e293b"
TEXT_SECONDARY = "#6b7280"
TEXT_MUTED = "#9ca3af"
SUCCESS = "#10b981"
WARNING = "#f59e0b"
ERROR = "#ef4444"
INFO = "#64b5f6"

_LAYER_COLOURS = {
    "Linear": TEAL, "Conv1d": INFO, "Conv2d": INFO, "Embedding": TERRACOTTA, "LayerNorm": WARNING, "RMSNorm": WARNING,
    "BatchNorm": WARNING, "Norm": WARNING, "Attention": SUCCESS, "Bias": TEXT_MUTED, "Tensor": TEXT_SECONDARY,
}
_SERIES = [TEAL, TERRACOTTA, INFO, SUCCESS, WARNING]


class AxonmlTheme:
    """Named styles; every method returns a ``rich`` style string."""

    @staticmethod
    def header() -> str: return f"bold {TEAL}"
    @staticmethod
    def title() -> str: return f"bold {CREAM}"
    @staticmethod
    def accent() -> str: return TERRACOTTA
    @staticmethod
    def selected() -> str: return f"bold {DARK_SLATE} on {TEAL_LIGHT}"
    @staticmethod
    def muted() -> str: return TEXT_MUTED
    @staticmethod
    def secondary() -> str: return TEXT_SECONDARY
    @staticmethod
    def border() -> str: return TEXT_SECONDARY
    @staticmethod
    def border_focused() -> str: return TEAL
    @staticmethod
    def tab_active() -> str: return f"bold {DARK_SLATE} on {TEAL}"
    @staticmethod
    def tab_inactive() -> str: return TEXT_MUTED
    @staticmethod
    def key() -> str: return f"bold {TERRACOTTA}"
    @staticmethod
    def success() -> str: return SUCCESS
    @staticmethod
    def warning() -> str: return WARNING
    @staticmethod
    def error() -> str: return f"bold {ERROR}"
    @staticmethod
    def info() -> str: return INFO
    @staticmethod
    def metric_value() -> str: return f"bold {TEAL_LIGHT}"

    @staticmethod
    def layer(kind: str) -> str:
        return _LAYER_COLOURS.get(kind, TEXT_SECONDARY)

    @staticmethod
    def series(i: int) -> str:
        return _SERIES[i % len(_SERIES)]

    @staticmethod
    def level(level: str) -> str:
        return {"info": INFO, "success": SUCCESS, "warning": WARNING, "error": f"bold {ERROR}"}.get(level, TEXT_MUTED)
