"""Server configuration from the environment.

Same variable names, defaults and parsing rules as the reference (envconfig/config.go:22-60 host,
:86-109 origins, :113-124 models dir, :129-164 keep-alive / load timeout, :199-212 log level,
:214-303 the remaining knobs, :311-372 ``AsMap``).  Knobs that only exist here are namespaced
``B200_*``.
"""
from __future__ import annotations

import ipaddress
import math
import os
import re
from dataclasses import dataclass
from urllib.parse import urlsplit

INF = math.inf


def var(key: str) -> str:
    """Environment value with surrounding whitespace and one layer of quotes removed."""
    return os.environ.get(key, "").strip().strip("\"'")


def _bool(key: str, default: bool = False) -> bool:
    s = var(key)
    if not s:
        return default
    if s.lower() in ("1", "t", "true", "yes", "on"):
        return True
    if s.lower() in ("0", "f", "false", "no", "off"):
        return False
    return True     # any other non-empty value enables the flag


def _uint(key: str, default: int) -> int:
    s = var(key)
    if s:
        try:
            n = int(s)
            if n >= 0:
                return n
        except ValueError:
            pass
    return default


_DUR = re.compile(r"([0-9]*\.?[0-9]+)(ns|us|µs|ms|s|m|h)")
_UNIT = {"ns": 1e-9, "us": 1e-6, "µs": 1e-6, "ms": 1e-3, "s": 1.0, "m": 60.0, "h": 3600.0}


def parse_duration(s: str) -> float | None:
    """Go ``time.ParseDuration`` subset ("5m", "1h30m", "-1s"); returns seconds or None."""
    s = s.strip()
    if not s:
        return None
    sign = 1.0
    if s[0] in "+-":
        sign = -1.0 if s[0] == "-" else 1.0
        s = s[1:]
    if s == "0":
        return 0.0
    pos, total = 0, 0.0
    for m in _DUR.finditer(s):
        if m.start() != pos:
            return None
        total += float(m.group(1)) * _UNIT[m.group(2)]
        pos = m.end()
    if pos != len(s) or pos == 0:
        return None
    return sign * total


def _duration(key: str, default: float, nonpositive_is_inf: bool) -> float:
    v = default
    s = var(key)
    if s:
        d = parse_duration(s)
        if d is not None:
            v = d
        else:
            try:
                v = float(int(s))
            except ValueError:
                pass
    if v < 0 or (nonpositive_is_inf and v <= 0):
        return INF
    return v


@dataclass
class HostURL:
    scheme: str
    host: str
    port: int
    path: str = ""

    @property
    def netloc(self) -> str:
        h = f"[{self.host}]" if ":" in self.host else self.host
        return f"{h}:{self.port}"

    def __str__(self) -> str:
        return f"{self.scheme}://{self.netloc}{('/' + self.path) if self.path else ''}"


def host() -> HostURL:
    """OLLAMA_HOST -> scheme/host/port; default http://127.0.0.1:11434."""
    default_port = 11434
    s = var("OLLAMA_HOST").strip()
    scheme, sep, hostport = s.partition("://")
    if not sep:
        scheme, hostport = "http", s
        if s == "ollama.com":
            scheme, hostport = "https", "ollama.com:443"
    elif scheme == "http":
        default_port = 80
    elif scheme == "https":
        default_port = 443
    hostport, _, path = hostport.partition("/")
    h, port = "127.0.0.1", default_port
    m = re.fullmatch(r"\[(.*)\]:(.*)|([^:]*):([^:]*)", hostport)
    if m:
        h = m.group(1) if m.group(1) is not None else m.group(3)
        ps = m.group(2) if m.group(2) is not None else m.group(4)
        try:            # an empty host (":1234") stays empty: every interface when listening, this machine when connecting
            port = int(ps)
            if not 0 <= port <= 65535:
                port = default_port
        except ValueError:
            port = default_port
    elif hostport:
        stripped = hostport.strip("[]")
        try:
            h = str(ipaddress.ip_address(stripped))
        except ValueError:
            h = hostport
    return HostURL(scheme, h, port, path)


def connectable_host() -> HostURL:
    """``host()`` for a client: the unspecified addresses a server may listen on (0.0.0.0, ::, empty) become the loopback
    address of the same family (envconfig/config.go ConnectableHost)."""
    u = host()
    if u.host in ("", "0.0.0.0"):
        u.host = "127.0.0.1"
    elif u.host == "::":
        u.host = "::1"
    return u


def allowed_origins() -> list[str]:
    origins = [o for o in var("OLLAMA_ORIGINS").split(",") if o]
    for o in ("localhost", "127.0.0.1", "0.0.0.0"):
        origins += [f"http://{o}", f"https://{o}", f"http://{o}:*", f"https://{o}:*"]
    origins += ["app://*", "file://*", "tauri://*", "vscode-webview://*", "vscode-file://*"]
    return origins


def models_dir() -> str:
    return var("OLLAMA_MODELS") or os.path.join(os.path.expanduser("~"), ".ollama", "models")


def keep_alive() -> float:
    """Seconds a model stays loaded; negative = forever (inf); default 5 minutes."""
    return _duration("OLLAMA_KEEP_ALIVE", 300.0, nonpositive_is_inf=False)


def load_timeout() -> float:
    return _duration("OLLAMA_LOAD_TIMEOUT", 300.0, nonpositive_is_inf=True)


def log_level() -> int:
    """Python logging level: INFO by default, DEBUG for OLLAMA_DEBUG=1/true, TRACE (5) for 2 and above; negative values
    lower the verbosity (-1 WARNING, -2 ERROR)."""
    s = var("OLLAMA_DEBUG")
    if not s:
        return 20
    if s.lower() in ("1", "t", "true"):
        return 10
    try:
        i = int(s)
    except ValueError:
        return 20
    if i < 0:
        return min(50, 20 - 10 * i)
    return 20 if i == 0 else (10 if i == 1 else 5)


def flash_attention(default: bool = True) -> bool:
    return _bool("OLLAMA_FLASH_ATTENTION", default)


def go_template(default: bool = False) -> bool:
    return _bool("OLLAMA_GO_TEMPLATE", default)


def debug_log_requests() -> bool:
    return _bool("OLLAMA_DEBUG_LOG_REQUESTS")


def kv_cache_type() -> str:
    return var("OLLAMA_KV_CACHE_TYPE")


def no_prune() -> bool:
    return _bool("OLLAMA_NOPRUNE")


def no_history() -> bool:
    return _bool("OLLAMA_NOHISTORY")


def sched_spread() -> bool:
    return _bool("OLLAMA_SCHED_SPREAD")


def _no_cloud_config() -> bool:
    """``disable_ollama_cloud`` of ~/.ollama/server.json; a missing or unreadable file counts as false."""
    import json
    try:
        with open(os.path.join(os.path.expanduser("~"), ".ollama", "server.json"), encoding="utf-8") as f:
            return bool(json.load(f).get("disable_ollama_cloud", False))
    except (OSError, ValueError, AttributeError):
        return False


def no_cloud() -> bool:
    """Cloud features are off when OLLAMA_NO_CLOUD is set or the server's config file disables them."""
    return _bool("OLLAMA_NO_CLOUD") or _no_cloud_config()


def no_cloud_source() -> str:
    """Which of the two switched cloud features off: "env", "config", "both" or "none"."""
    e, c = _bool("OLLAMA_NO_CLOUD"), _no_cloud_config()
    return "both" if e and c else "env" if e else "config" if c else "none"


def context_length() -> int:
    return _uint("OLLAMA_CONTEXT_LENGTH", 0)


def num_parallel() -> int:
    return _uint("OLLAMA_NUM_PARALLEL", 1)


def max_runners() -> int:
    return _uint("OLLAMA_MAX_LOADED_MODELS", 0)


def max_queue() -> int:
    return _uint("OLLAMA_MAX_QUEUE", 512)


def gpu_overhead() -> int:
    return _uint("OLLAMA_GPU_OVERHEAD", 0)


def llm_library() -> str:
    return var("OLLAMA_LLM_LIBRARY")


def cuda_visible_devices() -> str:
    return var("CUDA_VISIBLE_DEVICES")


# -- knobs of this runtime -----------------------------------------------------------------------
def tp_degree() -> int:
    """B200_TP: tensor-parallel degree used when a model does not fit (or to force a split); 0 = automatic."""
    return _uint("B200_TP", 0)


def pp_degree() -> int:
    """B200_PP: number of GPUs of a layer pipeline (consecutive layers on consecutive GPUs); 0 = only as the fallback of B200_TP."""
    return _uint("B200_PP", 0)


def replicas() -> int:
    """B200_REPLICAS: whole copies of a model on different GPUs, requests spread over them; 0 or 1 = one runner."""
    return _uint("B200_REPLICAS", 0)


def attn_splits() -> int:
    """B200_ATTN_SPLITS: upper bound of the split-K width of decode attention (CTAs per sequence and KV head)."""
    return max(1, _uint("B200_ATTN_SPLITS", 32))


def attn_split_len() -> int:
    """B200_ATTN_SPLIT_LEN: positions of allocated context per split of decode attention (splits = num_ctx / this, capped)."""
    return max(64, _uint("B200_ATTN_SPLIT_LEN", 512))


def comm_mode() -> str:
    """B200_COMM: nccl | p2p (fused peer-memory kernels, default) ."""
    return var("B200_COMM") or "p2p"


def device() -> str:
    """B200_DEVICE: auto | cpu | cuda[:N]."""
    return var("B200_DEVICE") or "auto"


def as_map() -> dict[str, tuple[object, str]]:
    """Every knob with its current value and description (``serve --help`` and the start-up log)."""
    return {
        "OLLAMA_DEBUG": (log_level(), "Show additional debug information (e.g. OLLAMA_DEBUG=1)"),
        "OLLAMA_FLASH_ATTENTION": (flash_attention(), "Enabled flash attention"),
        "OLLAMA_KV_CACHE_TYPE": (kv_cache_type(), "Quantization type for the K/V cache (default: f16)"),
        "OLLAMA_GPU_OVERHEAD": (gpu_overhead(), "Reserve a portion of VRAM per GPU (bytes)"),
        "OLLAMA_HOST": (str(host()), "IP Address for the ollama server (default 127.0.0.1:11434)"),
        "OLLAMA_KEEP_ALIVE": (keep_alive(), "The duration that models stay loaded in memory (default \"5m\")"),
        "OLLAMA_LLM_LIBRARY": (llm_library(), "Set LLM library to bypass autodetection"),
        "OLLAMA_LOAD_TIMEOUT": (load_timeout(), "How long to allow model loads to stall before giving up (default \"5m\")"),
        "OLLAMA_MAX_LOADED_MODELS": (max_runners(), "Maximum number of loaded models per GPU"),
        "OLLAMA_MAX_QUEUE": (max_queue(), "Maximum number of queued requests"),
        "OLLAMA_MODELS": (models_dir(), "The path to the models directory"),
        "OLLAMA_NOHISTORY": (no_history(), "Do not preserve readline history"),
        "OLLAMA_NOPRUNE": (no_prune(), "Do not prune model blobs on startup"),
        "OLLAMA_NUM_PARALLEL": (num_parallel(), "Maximum number of parallel requests"),
        "OLLAMA_ORIGINS": (allowed_origins(), "A comma separated list of allowed origins"),
        "OLLAMA_SCHED_SPREAD": (sched_spread(), "Always schedule model across all GPUs"),
        "OLLAMA_CONTEXT_LENGTH": (context_length(), "Context length to use unless otherwise specified (default: 4k/32k/256k based on VRAM)"),
        "OLLAMA_GO_TEMPLATE": (go_template(), "Render prompts with the Modelfile TEMPLATE when a model has one"),
        "OLLAMA_DEBUG_LOG_REQUESTS": (debug_log_requests(), "Log inference requests to disk for replay"),
        "OLLAMA_NO_CLOUD": (no_cloud(), "Disable cloud features"),
        "CUDA_VISIBLE_DEVICES": (cuda_visible_devices(), "Set which NVIDIA devices are visible"),
        "B200_TP": (tp_degree(), "Tensor-parallel degree (0 = automatic)"),
        "B200_PP": (pp_degree(), "GPUs of a layer pipeline (0 = only as the fallback of B200_TP)"),
        "B200_REPLICAS": (replicas(), "Data-parallel copies of a model, one per GPU (0 = one runner)"),
        "B200_ATTN_SPLITS": (attn_splits(), "Upper bound of the split-K width of decode attention"),
        "B200_ATTN_SPLIT_LEN": (attn_split_len(), "Positions of allocated context per split of decode attention"),
        "B200_ATTN_MMA": (var("B200_ATTN_MMA") or "auto", "Decode attention kernel: 1 tensor cores, 0 scalar, auto by model shape"),
        "B200_ATTN_PREFILL": (var("B200_ATTN_PREFILL") or "auto", "Prefill attention kernel: auto (tcgen05 where the shape allows), tc, mma"),
        "B200_ATTN_DECODE_STAGES": (var("B200_ATTN_DECODE_STAGES") or "auto", "Pipeline depth of the tensor-core decode attention: 2, 3, 4 or by launch size"),
        "B200_TC_DECODE_MIN": (var("B200_TC_DECODE_MIN") or "4", "Decode steps of at least this many sequences multiply 16-bit matrices on the tcgen05 GEMM (0 = never)"),
        "B200_MOE_STREAM_Q": (var("B200_MOE_STREAM_Q") or "1", "MoE prefill streams MXFP4 experts as they are when no 16-bit copy is resident (0 = expand per chunk)"),
        "B200_SK": (var("B200_SK") or "1", "Streaming decode GEMV for Q4_K / Q6_K / Q8_0 layers (0 = plane kernels)"),
        "B200_NVTX": (_bool("B200_NVTX"), "NVTX ranges around prefill chunks and decode steps"),
        "B200_NO_NATIVE": (_bool("B200_NO_NATIVE"), "Do not load the C++ host helpers (codecs, BPE merges)"),
        "B200_COMM": (comm_mode(), "Collective implementation: p2p (fused kernels) or nccl"),
        "B200_DEVICE": (device(), "Execution device: auto, cpu or cuda[:N]"),
    }
