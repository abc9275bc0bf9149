"""Human-readable sizes, counts and durations (format/ in the reference: bytes.go, format.go, time.go)."""
from __future__ import annotations


def human_bytes(n: float) -> str:
    """Decimal units as in listings: 999 B, 1.5 KB, 12 MB, 4.9 GB."""
    for unit, div in (("TB", 1e12), ("GB", 1e9), ("MB", 1e6), ("KB", 1e3)):
        if n >= div:
            v = n / div
            return f"{v:.1f} {unit}" if v < 10 else f"{v:.0f} {unit}"
    return f"{int(n)} B"


def human_bytes2(n: float) -> str:
    """Binary units as in memory logs: 457.0 MiB, 1.5 GiB."""
    for unit, div in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10)):
        if n >= div:
            return f"{n / div:.1f} {unit}"
    return f"{int(n)} B"


def human_number(n: int) -> str:
    """Parameter counts: 999, 1.50K, 137M, 8.03B, 1.2T."""
    if n >= 1e12:
        return f"{n / 1e12:.1f}T"
    if n >= 1e9:
        v = n / 1e9
        return f"{v:.2f}B" if v < 10 else f"{v:.1f}B"
    if n >= 1e6:
        v = n / 1e6
        return f"{v:.2f}M" if v < 10 else f"{v:.0f}M"
    if n >= 1e3:
        v = n / 1e3
        return f"{v:.2f}K" if v < 10 else f"{v:.0f}K"
    return str(int(n))


def human_duration(seconds: float) -> str:
    s = abs(seconds)
    for unit, div in (("year", 31536000), ("month", 2592000), ("week", 604800), ("day", 86400), ("hour", 3600), ("minute", 60)):
        if s >= div:
            n = int(s // div)
            return f"{n} {unit}{'s' if n != 1 else ''}"
    if s >= 1:
        n = int(s)
        return f"{n} second{'s' if n != 1 else ''}"
    return "Less than a second"
