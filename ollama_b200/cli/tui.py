"""Terminal pickers used by ``launch`` and ``run`` without arguments: a filterable list and a yes / no prompt.

The reference draws these with a terminal UI toolkit (cmd/tui/selector.go, confirm.go).  Here they are plain ANSI: on a
terminal the list is redrawn in place, arrow keys (or Ctrl-P / Ctrl-N) move, typing filters, Enter picks, Esc or Ctrl-C
cancels; when standard input is not a terminal (pipes, tests) the same functions read one line: an index, a name, or y / n.
The key handling is a pure function of (state, key), so it is tested without a terminal.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass, field
from typing import Callable, Sequence


@dataclass
class Item:
    name: str
    description: str = ""
    recommended: bool = False


class Cancelled(Exception):
    pass


@dataclass
class SelectorState:
    items: Sequence[Item]
    query: str = ""
    cursor: int = 0
    offset: int = 0
    height: int = 10
    visible: list[Item] = field(default_factory=list)

    def __post_init__(self):
        self.refilter()

    def refilter(self) -> None:
        q = self.query.lower()
        hits = [it for it in self.items if q in it.name.lower() or q in it.description.lower()]
        # names that start with the query come first, then the rest in their given order
        self.visible = sorted(hits, key=lambda it: not it.name.lower().startswith(q)) if q else list(hits)
        self.cursor = min(self.cursor, max(0, len(self.visible) - 1))
        self.offset = min(self.offset, self.cursor)

    def key(self, k: str) -> str | None:
        """Apply one key; returns "pick", "cancel" or None (keep going)."""
        if k in ("\r", "\n"):
            return "pick" if self.visible else None
        if k in ("\x1b", "\x03"):
            return "cancel"
        if k in ("up", "\x10"):
            self.cursor = max(0, self.cursor - 1)
        elif k in ("down", "\x0e"):
            self.cursor = min(max(0, len(self.visible) - 1), self.cursor + 1)
        elif k == "pgup":
            self.cursor = max(0, self.cursor - self.height)
        elif k == "pgdn":
            self.cursor = min(max(0, len(self.visible) - 1), self.cursor + self.height)
        elif k in ("\x7f", "\b"):
            self.query = self.query[:-1]
            self.refilter()
        elif len(k) == 1 and k.isprintable():
            self.query += k
            self.cursor = 0
            self.refilter()
        if self.cursor < self.offset:
            self.offset = self.cursor
        elif self.cursor >= self.offset + self.height:
            self.offset = self.cursor - self.height + 1
        return None

    def lines(self, title: str) -> list[str]:
        out = [f"{title} {self.query}\x1b[90m{'' if self.query else 'type to filter'}\x1b[0m"]
        window = self.visible[self.offset:self.offset + self.height]
        width = max((len(it.name) for it in window), default=0)
        for i, it in enumerate(window):
            mark = "\x1b[1m> " if self.offset + i == self.cursor else "  "
            tail = ("  \x1b[90m" + it.description + "\x1b[0m") if it.description else ""
            out.append(f"{mark}{it.name.ljust(width)}\x1b[0m{' (recommended)' if it.recommended else ''}{tail}")
        if not window:
            out.append("  \x1b[90m(no matches)\x1b[0m")
        more = len(self.visible) - self.offset - len(window)
        if more > 0:
            out.append(f"  \x1b[90m... and {more} more\x1b[0m")
        return out

    @property
    def current(self) -> Item:
        return self.visible[self.cursor]


def _read_key(fd: int) -> str:
    import os
    ch = os.read(fd, 1).decode(errors="ignore")
    if ch != "\x1b":
        return ch
    import select
    if not select.select([fd], [], [], 0.03)[0]:
        return "\x1b"
    seq = os.read(fd, 8).decode(errors="ignore")
    return {"[A": "up", "[B": "down", "[5~": "pgup", "[6~": "pgdn", "OA": "up", "OB": "down"}.get(seq, "")


def select(title: str, items: Sequence[Item], inp=None, out=None) -> str:
    """The name of the chosen item; raises :class:`Cancelled`."""
    inp, out = inp or sys.stdin, out or sys.stderr
    if not items:
        raise Cancelled("nothing to choose from")
    if not (hasattr(inp, "isatty") and inp.isatty()):
        for i, it in enumerate(items, 1):
            out.write(f"{i:3d}. {it.name}{'  ' + it.description if it.description else ''}\n")
        out.write(f"{title} ")
        out.flush()
        line = inp.readline()
        if not line:
            raise Cancelled("no selection")
        line = line.strip()
        if line.isdigit() and 1 <= int(line) <= len(items):
            return items[int(line) - 1].name
        names = [it.name for it in items]
        for exact in (line, line + ":latest"):          # a model name may be given without its default tag
            if line and exact in names:
                return exact
        hit = [n for n in names if n.startswith(line)] if line else []
        if len(hit) == 1:
            return hit[0]
        raise Cancelled(f"no such entry: {line!r}")
    import termios
    import tty
    fd = inp.fileno()
    saved = termios.tcgetattr(fd)
    st = SelectorState(items)
    drawn = 0
    try:
        tty.setcbreak(fd)
        out.write("\x1b[?25l")
        while True:
            lines = st.lines(title)
            out.write(("\x1b[%dA" % drawn if drawn else "") + "".join("\r\x1b[2K" + ln + "\n" for ln in lines) + "\x1b[J")
            out.flush()
            drawn = len(lines)
            verdict = st.key(_read_key(fd))
            if verdict == "pick":
                return st.current.name
            if verdict == "cancel":
                raise Cancelled("cancelled")
    finally:
        termios.tcsetattr(fd, termios.TCSADRAIN, saved)
        out.write("\x1b[?25h")
        out.flush()


def confirm(question: str, default: bool = False, inp=None, out=None) -> bool:
    inp, out = inp or sys.stdin, out or sys.stderr
    out.write(f"{question} [{'Y/n' if default else 'y/N'}] ")
    out.flush()
    line = inp.readline()
    if not line:
        return False
    ans = line.strip().lower()
    return default if not ans else ans in ("y", "yes")
