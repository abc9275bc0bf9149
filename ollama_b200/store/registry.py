"""Registry client: pull and push models over the OCI-distribution-style HTTP API.

Pull: ``GET /v2/<ns>/<model>/manifests/<tag>``, then every missing blob with ranged, resumable,
multi-part downloads (up to 16 parts of 100 MB - 1 GB, retried, digest verified; the reference's
policy in server/download.go:31,99-102,278-287,400-434) and finally the manifest is written.  Push:
``HEAD`` each blob, upload missing ones (``POST .../blobs/uploads/`` then ``PATCH``/``PUT``), then
``PUT`` the manifest (server/upload.go, server/images.go:931-1295).  Bearer-token challenges
(``WWW-Authenticate``) are answered with a token request signed by the installation's ed25519 key
(``ollama_b200/auth.py``).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import json
import os
import re
from typing import Any, Iterator

from . import manifest as M
from .names import Name, parse_name

NUM_PARTS = 16
MIN_PART = 100 << 20
MAX_PART = 1000 << 20
RETRIES = 6


class RegistryError(Exception):
    def __init__(self, msg: str, status: int = 500):
        super().__init__(msg)
        self.status = status


def _base(name: Name, insecure: bool) -> str:
    scheme = "http" if insecure or name.host.startswith(("localhost", "127.0.0.1")) else "https"
    return f"{scheme}://{name.host}/v2/{name.namespace}/{name.model}"


class _Session:
    def __init__(self):
        import requests
        self.s = requests.Session()
        self.token = ""

    def _token(self, ch: dict[str, str], url: str):
        """Answer a bearer challenge: the token request is signed with this installation's key when there is one
        (server/auth.go:53-100); the realm must be the host that issued the challenge, so that a signature never
        goes to a third party.  Without a key the request goes out unsigned (public namespaces)."""
        from urllib.parse import urlsplit

        from .. import auth
        turl = auth.challenge_url(ch["realm"], ch.get("service", ""), ch.get("scope", ""))
        if urlsplit(turl).netloc != urlsplit(url).netloc:
            raise RegistryError(f"realm host {urlsplit(turl).netloc!r} does not match original host {urlsplit(url).netloc!r}", 401)
        hdr = {}
        try:
            hdr["Authorization"] = auth.token_request_signature(turl)
        except auth.AuthError:
            pass
        return self.s.get(turl, headers=hdr, timeout=30)

    def request(self, method: str, url: str, **kw):
        import requests
        headers = dict(kw.pop("headers", {}) or {})
        if self.token:
            headers["Authorization"] = f"Bearer {self.token}"
        try:
            r = self.s.request(method, url, headers=headers, timeout=kw.pop("timeout", 60), **kw)
            if r.status_code == 401 and "www-authenticate" in r.headers and not kw.get("_retried"):
                ch = dict(re.findall(r'(\w+)="([^"]*)"', r.headers["www-authenticate"]))
                if ch.get("realm"):
                    tr = self._token(ch, url)
                    if tr is not None and tr.ok:
                        self.token = tr.json().get("token", "")
                        headers["Authorization"] = f"Bearer {self.token}"
                        r = self.s.request(method, url, headers=headers, timeout=60, **{k: v for k, v in kw.items() if k != "_retried"})
            return r
        except requests.RequestException as e:
            raise RegistryError(f"registry request failed: {e}", 502) from None


def _download_blob(sess: _Session, base: str, layer: M.Layer, progress) -> None:
    dst = M.blob_path(layer.digest)
    if os.path.exists(dst):
        progress(layer.size)
        return
    partial = dst + "-partial"
    size = layer.size
    part_size = min(max(size // NUM_PARTS, MIN_PART), MAX_PART) if size > MIN_PART else max(size, 1)
    parts = [(o, min(o + part_size, size)) for o in range(0, max(size, 1), part_size)] if size else []
    meta_path = partial + ".json"
    done: dict[str, int] = {}
    if os.path.exists(meta_path):
        try:
            done = json.load(open(meta_path))
        except ValueError:
            done = {}
    with open(partial, "ab"):
        pass
    url = f"{base}/blobs/{layer.digest}"

    def fetch(rng: tuple[int, int]) -> None:
        start, end = rng
        got = int(done.get(str(start), 0))
        if start + got >= end:
            progress(got)
            return
        progress(got)
        last: Exception | None = None
        for _ in range(RETRIES):
            try:
                r = sess.request("GET", url, headers={"Range": f"bytes={start + got}-{end - 1}"}, stream=True)
                if r.status_code not in (200, 206):
                    raise RegistryError(f"blob download failed with status {r.status_code}", r.status_code)
                with open(partial, "r+b") as f:
                    f.seek(start + got)
                    for chunk in r.iter_content(1 << 20):
                        f.write(chunk)
                        got += len(chunk)
                        done[str(start)] = got
                        progress(len(chunk))
                if start + got >= end:
                    return
            except (RegistryError, OSError) as e:
                last = e
        raise RegistryError(f"download of {layer.digest} failed: {last}", 502)

    with cf.ThreadPoolExecutor(max_workers=min(NUM_PARTS, max(1, len(parts)))) as ex:
        try:
            list(ex.map(fetch, parts))
        finally:
            with open(meta_path, "w") as f:
                json.dump(done, f)
    if M.sha256_file(partial) != layer.digest:
        os.unlink(partial)
        if os.path.exists(meta_path):
            os.unlink(meta_path)
        raise RegistryError(f"digest mismatch for {layer.digest}", 502)
    os.replace(partial, dst)
    if os.path.exists(meta_path):
        os.unlink(meta_path)


def pull_model(name: str, insecure: bool = False) -> Iterator[dict[str, Any]]:
    n = parse_name(name)
    if not n.valid:
        raise RegistryError(f"invalid model name {name!r}", 400)
    sess = _Session()
    base = _base(n, insecure)
    yield {"status": "pulling manifest"}
    r = sess.request("GET", f"{base}/manifests/{n.tag}", headers={"Accept": M.MT_MANIFEST})
    if r.status_code == 404:
        raise RegistryError("pull model manifest: file does not exist", 404)
    if not r.ok:
        raise RegistryError(f"pull model manifest: {r.status_code} {r.text[:200]}", 502)
    d = r.json()
    config = M.Layer.from_json(d.get("config", {}))
    layers = [M.Layer.from_json(x) for x in d.get("layers", [])]
    for layer in layers + [config]:
        total, completed = layer.size, 0
        short = layer.digest[7:19]
        updates: list[int] = []

        def progress(nbytes: int) -> None:
            updates.append(nbytes)

        yield {"status": f"pulling {short}", "digest": layer.digest, "total": total, "completed": 0}
        _download_blob(sess, base, layer, progress)
        completed = min(total, sum(updates))
        yield {"status": f"pulling {short}", "digest": layer.digest, "total": total, "completed": completed or total}
    yield {"status": "verifying sha256 digest"}
    yield {"status": "writing manifest"}
    M.write_manifest(n, config, layers)
    yield {"status": "success"}


def push_model(name: str, insecure: bool = False) -> Iterator[dict[str, Any]]:
    n = parse_name(name)
    if not n.valid:
        raise RegistryError(f"invalid model name {name!r}", 400)
    try:
        man = M.read_manifest(n)
    except M.StoreError as e:
        raise RegistryError(str(e), 404) from None
    sess = _Session()
    base = _base(n, insecure)
    yield {"status": "retrieving manifest"}
    for layer in man.layers + [man.config]:
        short = layer.digest[7:19]
        r = sess.request("HEAD", f"{base}/blobs/{layer.digest}")
        if r.status_code == 200:
            yield {"status": f"pushing {short}", "digest": layer.digest, "total": layer.size, "completed": layer.size}
            continue
        r = sess.request("POST", f"{base}/blobs/uploads/")
        if r.status_code not in (201, 202):
            raise RegistryError(f"push failed: upload could not start ({r.status_code})", 502)
        loc = r.headers.get("Location", "")
        if loc.startswith("/"):
            loc = base.split("/v2/")[0] + loc
        yield {"status": f"pushing {short}", "digest": layer.digest, "total": layer.size, "completed": 0}
        with open(layer.path(), "rb") as f:
            sep = "&" if "?" in loc else "?"
            r = sess.request("PUT", f"{loc}{sep}digest={layer.digest}", data=f, headers={"Content-Type": "application/octet-stream"}, timeout=3600)
        if r.status_code not in (201, 202, 204):
            raise RegistryError(f"push failed: blob upload returned {r.status_code}", 502)
        yield {"status": f"pushing {short}", "digest": layer.digest, "total": layer.size, "completed": layer.size}
    yield {"status": "pushing manifest"}
    r = sess.request("PUT", f"{base}/manifests/{n.tag}", data=json.dumps(man.to_json()), headers={"Content-Type": M.MT_MANIFEST})
    if r.status_code not in (200, 201, 202):
        raise RegistryError(f"push failed: manifest upload returned {r.status_code}", 502)
    yield {"status": "success"}
