"""Inference request logging for debugging (``OLLAMA_DEBUG_LOG_REQUESTS=1``).

Every inference request (generate, chat, embed and their OpenAI / Anthropic façades) is written to a fresh
directory under the system temp dir as ``<n>_<route>.json`` together with ``<n>_<route>.sh``, a curl command
that replays it against ``OLLAMA_HOST``.  Counterpart of server/inference_request_log.go:33-125.
"""
from __future__ import annotations

import itertools
import json
import logging
import os
import tempfile
import threading

from .. import envconfig

log = logging.getLogger("ollama_b200.server")
LOGGED = ("/api/generate", "/api/chat", "/api/embed", "/api/embeddings", "/v1/chat/completions", "/v1/completions", "/v1/embeddings",
          "/v1/responses", "/v1/messages")


class RequestLogger:
    def __init__(self, directory: str | None = None):
        self.enabled = envconfig.debug_log_requests()
        self.dir = directory
        self._n = itertools.count(1)
        self._lock = threading.Lock()

    def record(self, route: str, body: bytes) -> str | None:
        """Returns the path of the JSON file written, or None when logging is off or the route is not an inference route."""
        if not self.enabled or route not in LOGGED:
            return None
        with self._lock:
            if self.dir is None:
                self.dir = tempfile.mkdtemp(prefix="ollama-request-logs-")
                log.warning("request debug logging enabled; inference request bodies are written to %s", self.dir)
            n = next(self._n)
        stem = os.path.join(self.dir, f"{n:06d}_{route.strip('/').replace('/', '_')}")
        try:
            text = json.dumps(json.loads(body), indent=2)
        except ValueError:
            text = body.decode("utf-8", "replace")
        with open(stem + ".json", "w", encoding="utf-8") as f:
            f.write(text + "\n")
        with open(stem + ".sh", "w", encoding="utf-8") as f:
            f.write("#!/bin/sh\n"
                    f'curl -sS -X POST "${{OLLAMA_HOST:-{envconfig.connectable_host()}}}{route}" -H "Content-Type: application/json" '
                    f'--data-binary "@{os.path.basename(stem)}.json"\n')
        os.chmod(stem + ".sh", 0o755)
        return stem + ".json"
