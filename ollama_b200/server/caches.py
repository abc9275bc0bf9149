"""Process-local caches behind ``/api/tags`` and ``/api/show``.

Both answers are derived from files that rarely change, yet clients (editors, launchers) poll them.  The reference
keeps a list cache and a show cache (server/model_list_cache.go, server/model_show_cache.go); their local parts are:

* the list entry of a model is reused while its manifest file has the same modification time and size, so a poll
  stats the manifest files and reads only the ones that changed;
* a show response is stored per (canonical name, verbose) together with the manifest digest: a different digest
  replaces the entry.  Requests that overlay a system prompt or options bypass the cache because they change the
  response.  Nothing is written to disk: the caches live as long as the server process.
"""
from __future__ import annotations

import copy
import os
import threading
from typing import Any, Callable

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
