"""Logging, formatting and request-log helpers."""
import io
import json
import logging
import os

from ollama_b200.utils import format as F
from ollama_b200.utils import logutil


def test_human_formats():
    assert F.human_bytes(999) == "999 B" and F.human_bytes(1500) == "1.5 KB" and F.human_bytes(4.92e9) == "4.9 GB" and F.human_bytes(12e6) == "12 MB"
    assert F.human_bytes2(457 * (1 << 20)) == "457.0 MiB" and F.human_bytes2(1.5 * (1 << 30)) == "1.5 GiB"
    assert F.human_number(8_030_000_000) == "8.03B" and F.human_number(137_000_000) == "137M" and F.human_number(999) == "999"
    assert F.human_duration(90) == "1 minute" and F.human_duration(2 * 86400) == "2 days" and F.human_duration(0.2) == "Less than a second"


def test_key_value_log_lines_and_trace_level():
    buf = io.StringIO()
    logutil.setup(logutil.TRACE, stream=buf)
    log = logging.getLogger("ollama_b200.test")
    log.info('loaded "model"', extra={"vram": "4.9 GiB", "layers": 33})
    logutil.trace(log, "fine detail")
    lines = buf.getvalue().strip().split("\n")
    assert lines[0].startswith("time=") and " level=INFO " in lines[0] and 'msg="loaded \\"model\\""' in lines[0]
    assert 'vram="4.9 GiB"' in lines[0] and "layers=33" in lines[0] and "source=test_utils.py:" in lines[0]
    assert " level=TRACE " in lines[1]
    logutil.setup(logging.INFO, stream=buf)
    logutil.trace(log, "hidden")
    assert "hidden" not in buf.getvalue()


def test_request_logger_writes_body_and_replay_script(tmp_path, monkeypatch):
    from ollama_b200.server.request_log import RequestLogger
    monkeypatch.setenv("OLLAMA_DEBUG_LOG_REQUESTS", "1")
    rl = RequestLogger(str(tmp_path))
    assert rl.record("/api/tags", b"{}") is None                      # not an inference route
    p = rl.record("/api/chat", json.dumps({"model": "m", "messages": []}).encode())
    assert p and json.load(open(p))["model"] == "m"
    sh = open(p[:-5] + ".sh").read()
    assert "curl" in sh and "/api/chat" in sh and os.path.basename(p) in sh and os.access(p[:-5] + ".sh", os.X_OK)
    monkeypatch.setenv("OLLAMA_DEBUG_LOG_REQUESTS", "0")
    assert RequestLogger(str(tmp_path)).record("/api/chat", b"{}") is None
