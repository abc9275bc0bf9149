"""Logging set-up: key=value text lines and a TRACE level below DEBUG.

Counterpart of logutil/logutil.go in the reference (slog text handler, TRACE = -8 there; 5 here, below logging.DEBUG).
``OLLAMA_DEBUG`` selects the level: unset/0 INFO, 1/true DEBUG, 2 TRACE (envconfig.log_level).
"""
from __future__ import annotations

import logging
import os
import sys
import time

TRACE = 5
logging.addLevelName(TRACE, "TRACE")


class KeyValueFormatter(logging.Formatter):
    """``time=2026-01-01T00:00:00.000Z level=INFO source=sched.py:120 msg="..."`` plus any ``extra`` keys."""

    _skip = set(logging.LogRecord("", 0, "", 0, "", (), None).__dict__) | {"message", "asctime"}

    def format(self, r: logging.LogRecord) -> str:
        t = time.strftime("%Y-%m-%dT%H:%M:%S", time.gmtime(r.created)) + f".{int(r.msecs):03d}Z"
        msg = r.getMessage().replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n")
        out = f'time={t} level={r.levelname} source={os.path.basename(r.pathname)}:{r.lineno} msg="{msg}"'
        for k, v in r.__dict__.items():
            if k not in self._skip:
                s = str(v)
                out += f' {k}="{s}"' if (" " in s or not s) else f" {k}={s}"
        if r.exc_info:
            out += " " + self.formatException(r.exc_info).replace("\n", "\\n")
        return out


def setup(level: int | None = None, stream=None) -> None:
    from .. import envconfig
    h = logging.StreamHandler(stream or sys.stderr)
    h.setFormatter(KeyValueFormatter())
    root = logging.getLogger("ollama_b200")
    root.handlers[:] = [h]
    root.setLevel(level if level is not None else envconfig.log_level())
    root.propagate = False


def trace(logger: logging.Logger, msg: str, *args, **kw) -> None:
    if logger.isEnabledFor(TRACE):
        logger.log(TRACE, msg, *args, **kw)
