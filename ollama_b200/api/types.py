"""Wire-level types of the REST API.

Requests and responses travel as JSON objects with the same field names as the reference structs
(api/types.go:62-130 generate, :133-180 chat, :520-564 responses and metrics, :568-596 options).
Only the pieces with behaviour live here: option defaults and merging (``DefaultOptions``
api/types.go:1096-1123, ``Options.FromMap`` :991-1092), keep-alive durations (:1232-1271),
``think`` values (:1126-1230) and Modelfile ``PARAMETER`` formatting (:1274-1348).
"""
from __future__ import annotations

import math
from typing import Any

from .. import envconfig

# name -> (kind, default); kinds: int, float, bool?, int?, strs
OPTION_FIELDS: dict[str, tuple[str, Any]] = {
    # runtime sampling options
    "num_keep": ("int", 4), "seed": ("int", -1), "num_predict": ("int", -1), "top_k": ("int", 40), "top_p": ("float", 0.9),
    "min_p": ("float", 0.0), "typical_p": ("float", 1.0), "repeat_last_n": ("int", 64), "temperature": ("float", 0.8),
    "repeat_penalty": ("float", 1.0), "presence_penalty": ("float", 0.0), "frequency_penalty": ("float", 0.0), "stop": ("strs", None),
    # options that take effect when the model is loaded (a change forces a reload)
    "num_ctx": ("int", 0), "num_batch": ("int", 512), "num_gpu": ("int", -1), "main_gpu": ("int?", None), "use_mmap": ("bool?", None),
    "num_thread": ("int", 0), "draft_num_predict": ("int", 4),
}
RUNNER_FIELDS = ("num_ctx", "num_batch", "num_gpu", "main_gpu", "use_mmap", "num_thread", "draft_num_predict")
DEPRECATED_PARAMETERS = ("penalize_newline", "low_vram", "f16_kv", "logits_all", "vocab_only", "use_mlock", "mirostat", "mirostat_tau",
                         "mirostat_eta", "tfs_z", "numa")


class OptionError(ValueError):
    pass


def default_options() -> dict[str, Any]:
    o = {k: d for k, (_, d) in OPTION_FIELDS.items()}
    o["num_ctx"] = envconfig.context_length()
    o["stop"] = []
    return o


def options_from_map(opts: dict[str, Any], m: dict[str, Any] | None) -> dict[str, Any]:
    """Merge ``m`` into ``opts`` (in place) with the reference's type rules; unknown keys are ignored."""
    for key, val in (m or {}).items():
        spec = OPTION_FIELDS.get(key)
        if spec is None or val is None:
            continue
        kind = spec[0]
        if kind in ("int", "int?"):
            if isinstance(val, bool) or not isinstance(val, (int, float)) or val != val or val in (float("inf"), float("-inf")):
                raise OptionError(f'option "{key}" must be of type integer')
            opts[key] = int(val)
        elif kind == "float":
            if isinstance(val, bool) or not isinstance(val, (int, float)):
                raise OptionError(f'option "{key}" must be of type float32')
            opts[key] = float(val)
        elif kind == "bool?":
            if not isinstance(val, bool):
                raise OptionError(f'option "{key}" must be of type boolean')
            opts[key] = val
        elif kind == "strs":
            if isinstance(val, str):
                val = [val]
            if not isinstance(val, list):
                raise OptionError(f'option "{key}" must be of type array')
            if not all(isinstance(s, str) for s in val):
                raise OptionError(f'option "{key}" must be of an array of strings')
            opts[key] = list(val)
    return opts


def runner_options(opts: dict[str, Any]) -> dict[str, Any]:
    return {k: opts.get(k) for k in RUNNER_FIELDS}


def parse_keep_alive(v: Any) -> float | None:
    """JSON keep_alive: number of seconds or a Go duration string; negative means "forever" (inf).  None = not given."""
    if v is None:
        return None
    if isinstance(v, bool):
        raise ValueError("keep_alive must be a number or a duration string")
    if isinstance(v, (int, float)):
        return math.inf if v < 0 else float(v)
    if isinstance(v, str):
        d = envconfig.parse_duration(v)
        if d is None:
            try:
                d = float(v)
            except ValueError:
                raise ValueError(f"invalid duration {v!r}") from None
        return math.inf if d < 0 else d
    raise ValueError("keep_alive must be a number or a duration string")


THINK_LEVELS = ("low", "medium", "high", "max")


def parse_think(v: Any) -> bool | str | None:
    """``think``: bool or one of low/medium/high/max; None when absent."""
    if v is None:
        return None
    if isinstance(v, bool):
        return v
    if isinstance(v, str):
        if v in THINK_LEVELS:
            return v
        if v.lower() in ("true", "false"):
            return v.lower() == "true"
        raise ValueError(f'think value "{v}" is not supported; must be one of "high", "medium", "low", "max", true, or false')
    raise ValueError("think must be a boolean or a string")


def think_enabled(v: bool | str | None) -> bool:
    return bool(v) if not isinstance(v, str) else True


def format_parameters(params: dict[str, list[str]]) -> dict[str, Any]:
    """Modelfile PARAMETER strings -> typed option values (``stop`` keeps every occurrence)."""
    out: dict[str, Any] = {}
    for key, vals in params.items():
        if key in DEPRECATED_PARAMETERS:
            continue
        spec = OPTION_FIELDS.get(key)
        if spec is None:
            raise OptionError(f"unknown parameter '{key}'")
        kind = spec[0]
        last = vals[-1]
        try:
            if kind in ("int", "int?"):
                out[key] = int(last)
            elif kind == "float":
                out[key] = float(last)
            elif kind == "bool?":
                if last.lower() not in ("true", "false", "1", "0"):
                    raise ValueError(last)
                out[key] = last.lower() in ("true", "1")
            else:
                out[key] = list(vals)
        except ValueError:
            raise OptionError(f"invalid {'int' if kind.startswith('int') else 'float' if kind == 'float' else 'bool'} value [{' '.join(vals)}]") from None
    return out


def duration_ns(seconds: float) -> int:
    return int(seconds * 1e9)
