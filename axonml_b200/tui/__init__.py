"""Terminal user interface: Model / Data / Training / Graphs / Files / Help views with vim-style keys.

Parity: crates/axonml-tui (``App``, ``Tab``, ``AxonmlTheme``, the six views and ``run``).  The
reference draws with ratatui on a crossterm terminal and mostly shows demo data; this package draws
with ``rich``, reads real model files, datasets, folders and training logs, and follows a running
job's log.  Start it with ``axonml tui [--model F] [--data D] [--watch LOG]``."""
from .app import App, StatusLevel, StatusMessage, Tab, build_app, run
from .theme import AxonmlTheme
from .views import DataView, FilesView, GraphsView, HelpView, ModelView, TrainingView

__all__ = ["App", "StatusLevel", "StatusMessage", "Tab", "build_app", "run", "AxonmlTheme", "DataView", "FilesView", "GraphsView",
           "HelpView", "ModelView", "TrainingView"]
