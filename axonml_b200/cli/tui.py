"""``axonml tui``: starts the terminal interface of ``axonml_b200.tui``.

Parity: crates/axonml-cli/src/commands/tui.rs (``--model`` and ``--data`` open a file in their
views at start-up).  ``--watch`` follows a training log and ``--once`` prints every view once,
without a terminal, and exits."""
from __future__ import annotations

from ..tui import build_app
from ..tui.views.training import sparkline  # noqa: F401  (kept importable from here)


def cmd_tui(a) -> None:
    app = build_app(a.model, a.data, getattr(a, "watch", None))
    if a.once:
        print(app.run_once())
    else:
        app.run()
