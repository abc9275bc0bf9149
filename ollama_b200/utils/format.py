"""Human-readable sizes, counts and durations with the rounding rules of format/ in the reference (bytes.go:20-63,
format.go:15-34, time.go:12-78)."""
from __future__ import annotations

import datetime as dt


def human_bytes(n: float) -> str:
    """Decimal units as in listings: 999 B, 1.5 KB, 12 MB, 4.9 GB; whole values and values of 10 and more have no fraction."""
    n = int(n)
    for unit, div in (("TB", 10 ** 12), ("GB", 10 ** 9), ("MB", 10 ** 6), ("KB", 10 ** 3)):
        if n >= div:
            v = n / div
            return f"{int(v)} {unit}" if v >= 10 or v == int(v) else f"{v:.1f} {unit}"
    return f"{n} B"


def human_bytes2(n: float) -> str:
    """Binary units as in memory logs: 457.0 MiB, 1.5 GiB."""
    n = int(n)
    for unit, div in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10)):
        if n >= div:
            return f"{n / div:.1f} {unit}"
    return f"{n} B"


def human_number(n: int) -> str:
    """Parameter counts: 999, 1K, 125M, 500.55M, 8B, 2.9B."""
    n = int(n)
    if n >= 10 ** 9:
        v = n / 1e9
        return f"{v:.0f}B" if v == int(v) else f"{v:.1f}B"
    if n >= 10 ** 6:
        v = n / 1e6
        return f"{v:.0f}M" if v == int(v) else f"{v:.2f}M"
    if n >= 1000:
        return f"{n / 1e3:.0f}K"
    return str(n)


def human_duration(seconds: float) -> str:
    """Approximation of a span: "Less than a second", "About a minute", "3 hours", "2 days", "5 weeks", "7 months", "3 years"."""
    s = int(abs(seconds))
    if s < 1:
        return "Less than a second"
    if s < 60:
        return "1 second" if s == 1 else f"{s} seconds"
    minutes = s // 60
    if minutes < 60:
        return "About a minute" if minutes == 1 else f"{minutes} minutes"
    hours = int(abs(seconds) / 3600 + 0.5)
    if hours == 1:
        return "About an hour"
    if hours < 48:
        return f"{hours} hours"
    if hours < 24 * 7 * 2:
        return f"{hours // 24} days"
    if hours < 24 * 30 * 2:
        return f"{hours // 24 // 7} weeks"
    if hours < 24 * 365 * 2:
        return f"{hours // 24 // 30} months"
    return f"{int(abs(seconds) / 3600) // 24 // 365} years"


def human_time(t: dt.datetime | None, zero: str = "", now: dt.datetime | None = None) -> str:
    """"2 days ago" / "4 minutes from now"; more than twenty years ahead is "Forever"; ``None`` gives ``zero``."""
    if t is None:
        return zero
    now = now or dt.datetime.now(dt.timezone.utc)
    if t.tzinfo is None:
        t = t.replace(tzinfo=dt.timezone.utc)
    delta = (now - t).total_seconds()
    if int(delta / 3600 / 24 / 365) < -20:
        return "Forever"
    if delta < 0:
        return human_duration(-delta) + " from now"
    return human_duration(delta) + " ago"


def human_ago(iso: str) -> str:
    """``human_time`` of an RFC 3339 timestamp of the API; text that is no timestamp is returned as it is."""
    try:
        t = dt.datetime.fromisoformat(iso.replace("Z", "+00:00"))
    except (ValueError, AttributeError):
        return iso
    return human_time(t)
