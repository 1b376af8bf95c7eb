"""Key names and the decoder from raw terminal bytes.

Parity: crates/axonml-tui/src/event.rs (``poll_event`` with a timeout, ``read_event``).  The
reference receives decoded keys from crossterm; here the byte stream of a cbreak-mode terminal is
decoded directly: printable characters stand for themselves, control bytes and the CSI / SS3
sequences of the cursor keys map to the names below."""
from __future__ import annotations

import os
import select

UP, DOWN, LEFT, RIGHT = "up", "down", "left", "right"
ENTER, TAB, BACKTAB, BACKSPACE, ESC = "enter", "tab", "backtab", "backspace", "esc"
HOME, END, PAGE_UP, PAGE_DOWN = "home", "end", "pageup", "pagedown"

_CSI_FINAL = {"A": UP, "B": DOWN, "C": RIGHT, "D": LEFT, "Z": BACKTAB, "H": HOME, "F": END}
_CSI_TILDE = {"1": HOME, "7": HOME, "4": END, "8": END, "5": PAGE_UP, "6": PAGE_DOWN}


def decode(data: bytes) -> list[str]:
    """Every key contained in ``data`` (one read of the terminal can hold several)."""
    s = data.decode("utf-8", errors="replace")
    out, i = [], 0
    while i < len(s):
        c = s[i]
        if c == "\x1b":
            if i + 1 < len(s) and s[i + 1] in "[O":
                j = i + 2
                while j < len(s) and not ("@" <= s[j] <= "~"):
                    j += 1
                if j < len(s):
                    params, final = s[i + 2:j], s[j]
                    if final == "~":
                        name = _CSI_TILDE.get(params.split(";")[0])
                    else:
                        name = _CSI_FINAL.get(final)
                    if name:
                        out.append(name)
                    i = j + 1
                    continue
            out.append(ESC)
            i += 1
        elif c in "\r\n":
            out.append(ENTER)
            i += 1
        elif c == "\t":
            out.append(TAB)
            i += 1
        elif c in "\x7f\x08":
            out.append(BACKSPACE)
            i += 1
        elif c == "\x03":        # Ctrl-C quits like q
            out.append("q")
            i += 1
        elif c >= " ":
            out.append(c)
            i += 1
        else:
            i += 1
    return out


def poll(fd: int, timeout: float) -> bool:
    """True when input is waiting on ``fd``."""
    r, _, _ = select.select([fd], [], [], timeout)
    return bool(r)


def read_keys(fd: int, timeout: float) -> list[str]:
    """Keys typed within ``timeout`` seconds (possibly none)."""
    if not poll(fd, timeout):
        return []
    data = os.read(fd, 64)
    # an escape sequence may arrive in two reads
    if data.endswith(b"\x1b") and poll(fd, 0.02):
        data += os.read(fd, 16)
    return decode(data)
