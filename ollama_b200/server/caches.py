"""Process-local caches behind ``/api/tags`` and ``/api/show``.

Both answers are derived from files that rarely change, yet clients (editors, launchers) poll them.  The reference
keeps a list cache and a show cache (server/model_list_cache.go, server/model_show_cache.go); their local parts are:

* the list entry of a model is reused while its manifest file has the same modification time and size, so a poll
  stats the manifest files and reads only the ones that changed;
* a show response is stored per (canonical name, verbose) together with the manifest digest: a different digest
  replaces the entry.  Requests that overlay a system prompt or options bypass the cache because they change the
  response.  Nothing is written to disk: the caches live as long as the server process;
* the model object an inference request works with (layers resolved to paths, template, parameters, GGUF metadata,
  capabilities) is kept per canonical name with the manifest digest as freshness bound, and every request gets its own
  shallow copy (server/model_inference_cache.go:14-125).  Without it each request re-reads the manifest's layers and
  re-parses the GGUF header, vocabulary included;
* model recommendations (server/model_recommendations.go): a built-in list, replaced by the last snapshot on disk and by
  what the recommendation service answers, fetched in the background at most once per cool-down while reads are served
  from what is there (stale-while-revalidate), with a stepped back-off after failures and no fetch at all when cloud
  features are off.
"""
from __future__ import annotations

import copy
import json
import logging
import os
import threading
import time
from typing import Any, Callable

from .. import envconfig

from ..store import manifest as M


class ModelListCache:
    def __init__(self):
        self._lock = threading.Lock()
        self._entries: dict[str, tuple[tuple[int, int], dict[str, Any]]] = {}
        self.hits = self.misses = 0

    def list(self, build: Callable[[Any, Any], dict[str, Any]]) -> list[dict[str, Any]]:
        """``build(name, manifest)`` makes the entry of one model; called only for new or changed manifests."""
        out, seen = [], set()
        for n, path in M.manifest_names():
            try:
                st = os.stat(path)
            except OSError:
                continue
            stamp = (st.st_mtime_ns, st.st_size)
            seen.add(path)
            with self._lock:
                hit = self._entries.get(path)
            if hit is not None and hit[0] == stamp:
                self.hits += 1
                out.append(copy.deepcopy(hit[1]))
                continue
            try:
                entry = build(n, M.read_manifest(n))
            except (M.StoreError, ValueError, OSError):
                continue
            self.misses += 1
            with self._lock:
                self._entries[path] = (stamp, entry)
            out.append(copy.deepcopy(entry))
        with self._lock:
            for path in [p for p in self._entries if p not in seen]:      # deleted models
                del self._entries[path]
        return out


class ModelShowCache:
    def __init__(self, max_entries: int = 256):
        self._lock = threading.Lock()
        self._entries: dict[tuple[str, bool], tuple[str, dict[str, Any]]] = {}
        self.max_entries = max_entries
        self.hits = self.misses = 0

    @staticmethod
    def cacheable(req: dict[str, Any]) -> bool:
        return not req.get("system") and not req.get("options") and not req.get("template")

    def get(self, name: str, verbose: bool, digest: str) -> dict[str, Any] | None:
        with self._lock:
            hit = self._entries.get((name, verbose))
        if hit is not None and hit[0] == digest and digest:
            self.hits += 1
            return copy.deepcopy(hit[1])
        self.misses += 1
        return None

    def put(self, name: str, verbose: bool, digest: str, response: dict[str, Any]) -> None:
        if not digest:
            return
        with self._lock:
            if len(self._entries) >= self.max_entries and (name, verbose) not in self._entries:
                self._entries.pop(next(iter(self._entries)))                # oldest insertion
            self._entries[(name, verbose)] = (digest, copy.deepcopy(response))

    def drop(self, name: str) -> None:
        with self._lock:
            for k in [k for k in self._entries if k[0] == name]:
                del self._entries[k]


class InferenceModelCache:
    def __init__(self, load: Callable[[str], Any] | None = None):
        from ..store.model import get_model
        self.load = load or get_model
        self._lock = threading.Lock()
        self._entries: dict[tuple[str, bool], tuple[str, Any]] = {}
        self._loading: dict[tuple[str, bool], threading.Lock] = {}
        self.hits = self.misses = 0

    def get(self, name: str) -> Any:
        """The model named ``name`` as of its current manifest; raises what ``load`` raises (ModelNotFound)."""
        from ..store.model import ModelNotFound
        from ..store.names import parse_name
        n = parse_name(name)
        if not n.valid:
            raise ModelNotFound(name)
        try:
            digest = M.read_manifest(n).digest
        except (M.StoreError, ValueError):
            self.drop(str(n))
            raise ModelNotFound(name) from None
        key = (str(n), bool(envconfig.go_template()))
        with self._lock:
            hit = self._entries.get(key)
            if hit is not None and hit[0] == digest:
                self.hits += 1
                return self._clone(hit[1])
            gate = self._loading.setdefault(key, threading.Lock())
        with gate:                                   # one load per model at a time; the others wait and take its result
            with self._lock:
                hit = self._entries.get(key)
                if hit is not None and hit[0] == digest:
                    self.hits += 1
                    return self._clone(hit[1])
            m = self.load(name)
            m.kv()
            m._caps = m.capabilities()
            with self._lock:
                self.misses += 1
                self._entries[key] = (m.digest, m)
        return self._clone(m)

    @staticmethod
    def _clone(m: Any) -> Any:
        c = copy.copy(m)                             # the GGUF metadata is shared and read-only; what requests edit is copied
        for attr in ("adapter_paths", "projector_paths", "draft_paths", "license", "messages"):
            setattr(c, attr, list(getattr(m, attr)))
        c.options, c.config = dict(m.options), copy.deepcopy(m.config)
        return c

    def drop(self, name: str) -> None:
        with self._lock:
            for key in [k for k in self._entries if k[0] == name]:
                del self._entries[key]


log = logging.getLogger("ollama_b200.caches")
GB = 1000 ** 3
RECOMMENDATIONS_URL = "https://ollama.com/api/experimental/model-recommendations"
# what this engine runs, sized for one B200 and for a node of eight
DEFAULT_RECOMMENDATIONS: list[dict[str, Any]] = [
    {"model": "gpt-oss:120b", "description": "Reasoning and agentic tool use; MXFP4 experts, fits one B200", "vram_bytes": 66 * GB},
    {"model": "qwen3:235b-a22b", "description": "Mixture-of-experts reasoning and coding across the GPUs of a node", "vram_bytes": 143 * GB},
    {"model": "llama3.1:70b", "description": "General chat and instruction following, one GPU or tensor-parallel", "vram_bytes": 43 * GB},
    {"model": "gpt-oss:20b", "description": "Reasoning and tool use at low latency", "vram_bytes": 14 * GB},
    {"model": "qwen3:8b", "description": "Reasoning and coding, many parallel requests per GPU", "vram_bytes": 6 * GB},
    {"model": "gemma3:27b", "description": "General chat with long context", "vram_bytes": 18 * GB},
]
_REC_FIELDS = {"model": str, "description": str, "context_length": int, "max_output_tokens": int, "vram_bytes": int, "required_plan": str}


def validate_recommendations(items: Any) -> list[dict[str, Any]]:
    """Entries as the API serves them: known fields of the right kind only, a model name is required, duplicates dropped."""
    if not isinstance(items, list):
        raise ValueError("recommendations must be a list")
    out, seen = [], set()
    for it in items:
        if not isinstance(it, dict) or not isinstance(it.get("model"), str) or not it["model"].strip():
            raise ValueError("a recommendation needs a model name")
        rec = {}
        for k, kind in _REC_FIELDS.items():
            v = it.get(k)
            if v is None or v == "" or v == 0:
                continue
            if isinstance(v, bool) or not isinstance(v, kind) or (kind is int and v < 0):
                raise ValueError(f"recommendation field {k!r} has the wrong type")
            rec[k] = v.strip() if kind is str else v
        if rec["model"] in seen:
            continue
        seen.add(rec["model"])
        rec.setdefault("description", "")
        out.append(rec)
    if not out:
        raise ValueError("no recommendations")
    return out


class RecommendationsCache:
    BACKOFF = (300.0, 900.0, 3600.0, 4 * 3600.0)      # waits after 1, 2, 3, 4+ failures in a row
    REFRESH = 4 * 3600.0                              # wait after a success
    READ_COOLDOWN = 5.0                               # a read triggers at most one background fetch per this many seconds

    def __init__(self, fetch: Callable[[], Any] | None = None, snapshot_path: str | None = None, now: Callable[[], float] = time.monotonic):
        self.fetch = fetch or self._http_fetch
        self.snapshot_path = snapshot_path or os.path.join(os.path.expanduser("~"), ".ollama", "cache", "model-recommendations.json")
        self.now = now
        self._lock = threading.Lock()
        self._recs = copy.deepcopy(DEFAULT_RECOMMENDATIONS)
        self.source = "default"
        self._refreshing = False
        self._next_ok = 0.0
        self.failures = 0
        self._load_snapshot()

    def get(self) -> list[dict[str, Any]]:
        with self._lock:
            return copy.deepcopy(self._recs)

    def get_swr(self, background: bool = True) -> list[dict[str, Any]]:
        """What is cached now; a refresh is started behind the reader's back when none is running and the cool-down allows."""
        recs = self.get()
        with self._lock:
            start = not self._refreshing and self.now() >= self._next_ok
            if start:
                self._refreshing = True
        if start:
            if background:
                threading.Thread(target=self._refresh, daemon=True).start()
            else:
                self._refresh()
        return recs

    def _refresh(self) -> None:
        wait = self.READ_COOLDOWN
        try:
            if envconfig.no_cloud():
                self.failures = 0
                return                                # cloud features off: the built-in list (or the snapshot) is the answer
            recs = validate_recommendations(self.fetch())
            with self._lock:
                self._recs, self.source = recs, "remote"
            self.failures = 0
            wait = self.REFRESH
            self._save_snapshot(recs)
        except Exception as e:                        # network, status, JSON or validation: keep what we have, try later
            self.failures += 1
            wait = self.BACKOFF[min(self.failures, len(self.BACKOFF)) - 1]
            log.warning("model recommendations refresh failed (%d in a row): %s", self.failures, e)
        finally:
            with self._lock:
                self._refreshing = False
                self._next_ok = self.now() + wait

    def _load_snapshot(self) -> None:
        try:
            with open(self.snapshot_path, encoding="utf-8") as f:
                recs = validate_recommendations(json.load(f).get("recommendations"))
        except (OSError, ValueError, AttributeError):
            return
        self._recs, self.source = recs, "snapshot"

    def _save_snapshot(self, recs: list[dict[str, Any]]) -> None:
        try:
            os.makedirs(os.path.dirname(self.snapshot_path), exist_ok=True)
            tmp = self.snapshot_path + ".tmp"
            with open(tmp, "w", encoding="utf-8") as f:
                json.dump({"recommendations": recs}, f)
            os.replace(tmp, self.snapshot_path)
        except OSError as e:
            log.warning("could not store the model recommendations snapshot: %s", e)

    @staticmethod
    def _http_fetch() -> Any:
        import urllib.request
        req = urllib.request.Request(RECOMMENDATIONS_URL, headers={"Accept": "application/json"})
        with urllib.request.urlopen(req, timeout=3.0) as r:
            return json.load(r).get("recommendations")
