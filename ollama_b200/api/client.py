"""HTTP client of the REST API (the transport of every CLI command except ``serve``).

Mirrors the role of api/client.go in the reference: JSON requests, NDJSON streaming responses
(one JSON object per line, errors as ``{"error": ...}``), base URL from ``OLLAMA_HOST``.  Only the
standard library is used so that the CLI starts fast.
"""
from __future__ import annotations

import json
import urllib.error
import urllib.request
from typing import Any, Iterator

from .. import envconfig
from ..version import VERSION


class ResponseError(Exception):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status, self.message = status, message


class Client:
    def __init__(self, base: str | None = None, timeout: float | None = None):
        self.base = (base or str(envconfig.connectable_host())).rstrip("/")
        self.timeout = timeout

    # -- transport ----------------------------------------------------------------------------------
    def _open(self, method: str, path: str, body: Any = None, raw: bytes | None = None):
        data = raw if raw is not None else (json.dumps(body).encode() if body is not None else None)
        req = urllib.request.Request(self.base + path, data=data, method=method)
        req.add_header("Accept", "application/x-ndjson")
        req.add_header("User-Agent", f"ollama-b200/{VERSION}")
        if body is not None:
            req.add_header("Content-Type", "application/json")
        elif raw is not None:
            req.add_header("Content-Type", "application/octet-stream")
        try:
            return urllib.request.urlopen(req, timeout=self.timeout)
        except urllib.error.HTTPError as e:
            text = e.read().decode("utf-8", "replace")
            try:
                msg = json.loads(text).get("error", text)
            except (ValueError, AttributeError):
                msg = text
            raise ResponseError(e.code, msg or e.reason) from None
        except urllib.error.URLError as e:
            raise ConnectionError(f"could not connect to a server at {self.base}: {e.reason}") from None

    def request(self, method: str, path: str, body: Any = None) -> Any:
        with self._open(method, path, body) as r:
            text = r.read()
        return json.loads(text) if text.strip() else None

    def stream(self, method: str, path: str, body: Any = None) -> Iterator[dict[str, Any]]:
        with self._open(method, path, body) as r:
            for line in r:
                line = line.strip()
                if not line:
                    continue
                obj = json.loads(line)
                if isinstance(obj, dict) and obj.get("error"):
                    raise ResponseError(obj.get("status", 500) if isinstance(obj.get("status"), int) else 500, obj["error"])
                yield obj

    # -- endpoints ----------------------------------------------------------------------------------
    def heartbeat(self) -> bool:
        try:
            with self._open("HEAD", "/"):
                return True
        except (ConnectionError, ResponseError):
            return False

    def version(self) -> str:
        return self.request("GET", "/api/version")["version"]

    def generate(self, **req) -> Iterator[dict[str, Any]]:
        return self.stream("POST", "/api/generate", req)

    def chat(self, **req) -> Iterator[dict[str, Any]]:
        return self.stream("POST", "/api/chat", req)

    def embed(self, **req) -> dict[str, Any]:
        return self.request("POST", "/api/embed", req)

    def embeddings(self, **req) -> dict[str, Any]:
        """Legacy single-prompt embedding route (api/client.go Embeddings)."""
        return self.request("POST", "/api/embeddings", req)

    def status(self) -> dict[str, Any]:
        """Cloud status of the server (api/client.go CloudStatusExperimental)."""
        return self.request("GET", "/api/status")

    def tokenize(self, **req) -> dict[str, Any]:
        return self.request("POST", "/api/tokenize", req)

    def detokenize(self, **req) -> dict[str, Any]:
        return self.request("POST", "/api/detokenize", req)

    def list(self) -> dict[str, Any]:
        return self.request("GET", "/api/tags")

    def ps(self) -> dict[str, Any]:
        return self.request("GET", "/api/ps")

    def show(self, model: str, verbose: bool = False) -> dict[str, Any]:
        return self.request("POST", "/api/show", {"model": model, "verbose": verbose})

    def copy(self, source: str, destination: str) -> None:
        self.request("POST", "/api/copy", {"source": source, "destination": destination})

    def delete(self, model: str) -> None:
        self.request("DELETE", "/api/delete", {"model": model})

    def pull(self, model: str, insecure: bool = False) -> Iterator[dict[str, Any]]:
        return self.stream("POST", "/api/pull", {"model": model, "insecure": insecure})

    def push(self, model: str, insecure: bool = False) -> Iterator[dict[str, Any]]:
        return self.stream("POST", "/api/push", {"model": model, "insecure": insecure})

    def create(self, **req) -> Iterator[dict[str, Any]]:
        return self.stream("POST", "/api/create", req)

    def blob_exists(self, digest: str) -> bool:
        try:
            with self._open("HEAD", f"/api/blobs/{digest}"):
                return True
        except ResponseError as e:
            if e.status == 404:
                return False
            raise

    def create_blob(self, digest: str, data: bytes) -> None:
        with self._open("POST", f"/api/blobs/{digest}", raw=data):
            pass
