"""Line editing and history for the interactive prompt.

The reference carries its own terminal line editor (readline/readline.go, buffer.go) with a history file of the last 100
entries under ``~/.ollama/history`` that is rewritten after every line (readline/history.go:24-103) and switched off by
``OLLAMA_NOHISTORY``.  Python ships GNU readline bindings, so the editor itself (cursor keys, Ctrl-A/E/K/W, reverse search,
bracketed paste) comes from there; this module adds what is specific to the prompt: the history file with its limit, Tab
completion of the slash commands, and a plain ``input()`` fallback where the module or a terminal is missing.
"""
from __future__ import annotations

import os
import sys

from .. import envconfig

LIMIT = 100
COMMANDS = ("/set", "/show", "/load", "/save", "/clear", "/bye", "/exit", "/help", "/?")
SET_WORDS = ("parameter", "system", "history", "nohistory", "wordwrap", "nowordwrap", "format", "noformat", "verbose", "quiet", "think", "nothink")
SHOW_WORDS = ("info", "license", "modelfile", "parameters", "system", "template")


def history_path() -> str:
    return os.path.join(os.path.expanduser("~"), ".ollama", "history")


class History:
    """The entries of the history file, oldest first; ``add`` appends, drops what exceeds the limit and saves."""

    def __init__(self, path: str | None = None, limit: int = LIMIT, enabled: bool | None = None):
        self.path = path or history_path()
        self.limit = limit
        self.enabled = (not envconfig.no_history()) if enabled is None else enabled
        self.entries: list[str] = []
        if self.enabled:
            try:
                with open(self.path, encoding="utf-8") as f:
                    self.entries = [ln.rstrip("\n") for ln in f if ln.strip()][-limit:]
            except OSError:
                pass

    def add(self, line: str) -> None:
        line = line.replace("\n", " ").strip()
        if not line or not self.enabled or (self.entries and self.entries[-1] == line):
            return
        self.entries.append(line)
        del self.entries[:-self.limit]
        self.save()

    def save(self) -> None:
        try:
            os.makedirs(os.path.dirname(self.path), exist_ok=True)
            tmp = self.path + ".tmp"
            with open(tmp, "w", encoding="utf-8") as f:
                f.write("".join(e + "\n" for e in self.entries))
            os.replace(tmp, self.path)
        except OSError:
            pass                                    # a read-only home directory costs the history, not the session

    def clear(self) -> None:
        self.entries.clear()
        self.save()


def complete(text: str, line: str) -> list[str]:
    """Candidates for the word ``text`` at the end of ``line``: slash commands first, then the words ``/set`` and ``/show`` take."""
    words = line[:len(line) - len(text)].split()
    if not words:
        return [c + " " for c in COMMANDS if c.startswith(text)] if text.startswith("/") else []
    if len(words) == 1 and words[0] == "/set":
        return [w + " " for w in SET_WORDS if w.startswith(text)]
    if len(words) == 1 and words[0] == "/show":
        return [w for w in SHOW_WORDS if w.startswith(text)]
    return []


class LineEditor:
    """``read(prompt)`` returns one edited line (raises EOFError / KeyboardInterrupt like ``input``) and records it."""

    def __init__(self, history: History | None = None):
        self.history = history or History()
        self.rl = None
        if sys.stdin.isatty():
            try:
                import readline
                self.rl = readline
            except ImportError:
                pass
        if self.rl is not None:
            rl = self.rl
            rl.set_auto_history(False)
            rl.clear_history()
            for e in self.history.entries:
                rl.add_history(e)
            rl.set_completer_delims(" \t")
            rl.set_completer(self._completer)
            rl.parse_and_bind("tab: complete")
            rl.parse_and_bind("set enable-bracketed-paste on")

    def _completer(self, text: str, state: int):
        line = self.rl.get_line_buffer()[:self.rl.get_endidx()]
        cands = complete(text, line)
        return cands[state] if state < len(cands) else None

    def read(self, prompt: str, record: bool = True) -> str:
        line = input(prompt)
        if record and line.strip():
            if self.rl is not None and self.history.enabled:
                self.rl.add_history(line)
            self.history.add(line)
        return line

    def set_enabled(self, on: bool) -> None:
        self.history.enabled = on
