"""Logging, formatting and request-log helpers."""
import io
import json
import logging
import os

from ollama_b200.utils import format as F
from ollama_b200.utils import logutil


def test_human_formats():
    """Tables of format/bytes_test.go, format_test.go and time_test.go of the reference."""
    import datetime as dt
    for n, want in {0: "0 B", 1: "1 B", 999: "999 B", 1000: "1 KB", 1500: "1.5 KB", 999999: "999 KB", 1000000: "1 MB", 1500000: "1.5 MB",
                    999999999: "999 MB", 10 ** 9: "1 GB", 1500000000: "1.5 GB", 999999999999: "999 GB", 10 ** 12: "1 TB", 1500000000000: "1.5 TB",
                    1999999999999: "2.0 TB", 1234: "1.2 KB", 1234567: "1.2 MB", 1234567890: "1.2 GB", 4.92e9: "4.9 GB", 12e6: "12 MB"}.items():
        assert F.human_bytes(n) == want
    for n, want in {0: "0 B", 1023: "1023 B", 1024: "1.0 KiB", 1536: "1.5 KiB", 1048575: "1024.0 KiB", 1048576: "1.0 MiB", 1073741823: "1024.0 MiB",
                    1073741824: "1.0 GiB", 1610612736: "1.5 GiB", 2147483648: "2.0 GiB", 457 * (1 << 20): "457.0 MiB"}.items():
        assert F.human_bytes2(n) == want
    for n, want in {0: "0", 999: "999", 1000: "1K", 1001: "1K", 10 ** 6: "1M", 125000000: "125M", 500500000: "500.50M", 500550000: "500.55M",
                    10 ** 9: "1B", 2800000000: "2.8B", 2850000000: "2.9B", 10 ** 12: "1000B", 8_030_000_000: "8.0B"}.items():
        assert F.human_number(n) == want
    for s, want in {0.2: "Less than a second", 1: "1 second", 59: "59 seconds", 90: "About a minute", 150: "2 minutes", 3600: "About an hour",
                    5 * 3600: "5 hours", 2 * 86400: "2 days", 20 * 86400: "2 weeks", 90 * 86400: "3 months", 3 * 365 * 86400: "3 years"}.items():
        assert F.human_duration(s) == want
    now = dt.datetime(2026, 1, 1, tzinfo=dt.timezone.utc)
    assert F.human_time(None, "never") == "never"
    assert F.human_time(now + dt.timedelta(hours=48), now=now) == "2 days from now" and F.human_time(now - dt.timedelta(hours=48), now=now) == "2 days ago"
    assert F.human_time(now + dt.timedelta(milliseconds=800), now=now) == "Less than a second from now"
    assert F.human_time(now + dt.timedelta(days=365 * 200), now=now) == "Forever"
    assert F.human_ago("not a time") == "not a time" and F.human_ago("2001-01-01T00:00:00Z").endswith("years ago")


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
