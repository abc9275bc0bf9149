"""Registry client against an in-process registry: push, signed token requests, ranged resumable pull, digest checks."""
import base64
import hashlib
import http.server
import json
import os
import threading
from urllib.parse import parse_qs, urlsplit

import pytest

from ollama_b200 import auth
from ollama_b200.store import manifest as M
from ollama_b200.store import registry as reg
from ollama_b200.store.names import parse_name


class _Registry(http.server.BaseHTTPRequestHandler):
    blobs: dict = {}
    manifests: dict = {}
    seen: dict = {"signed": [], "ranges": []}
    pubkey_blob = ""
    protocol_version = "HTTP/1.1"

    def log_message(self, *a):
        pass

    def _send(self, code, body=b"", headers=None):
        self.send_response(code)
        for k, v in (headers or {}).items():
            self.send_header(k, v)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        if self.command != "HEAD":
            self.wfile.write(body)

    def _authorised(self):
        if self.headers.get("Authorization") == "Bearer sesame":
            return True
        host = self.headers["Host"]
        self._send(401, b"", {"WWW-Authenticate": f'Bearer realm="http://{host}/token",service="reg",scope="repository:me/thing:pull repository:me/thing:push"'})
        return False

    def _token(self):
        """Verifies the signature the way a registry would: over METHOD,URL,base64(hex(sha256(empty)))."""
        from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PublicKey
        q = parse_qs(urlsplit(self.path).query)
        ok = q.get("service") == ["reg"] and len(q.get("scope", [])) == 2 and q.get("ts") and q.get("nonce")
        hdr = self.headers.get("Authorization", "")
        blob, _, sig = hdr.partition(":")
        if ok and blob == self.pubkey_blob and sig:
            raw = base64.b64decode(blob)
            key = Ed25519PublicKey.from_public_bytes(raw[-32:])           # ssh blob: string "ssh-ed25519", string key
            url = f"http://{self.headers['Host']}{self.path}"
            empty = base64.b64encode(hashlib.sha256(b"").hexdigest().encode()).decode()
            key.verify(base64.b64decode(sig), f"GET,{url},{empty}".encode())    # raises on a bad signature
            self.seen["signed"].append(url)
            return self._send(200, json.dumps({"token": "sesame"}).encode(), {"Content-Type": "application/json"})
        self._send(403, b"unknown key")

    def do_GET(self):
        path = urlsplit(self.path).path
        if path == "/token":
            return self._token()
        if not self._authorised():
            return
        if "/manifests/" in path:
            m = self.manifests.get(path)
            return self._send(200, m, {"Content-Type": M.MT_MANIFEST}) if m else self._send(404, b"{}")
        digest = path.rsplit("/", 1)[1]
        data = self.blobs.get(digest)
        if data is None:
            return self._send(404)
        rng = self.headers.get("Range")
        if rng:
            a, b = rng.split("=")[1].split("-")
            self.seen["ranges"].append((int(a), int(b)))
            return self._send(206, data[int(a):int(b) + 1])
        self._send(200, data)

    do_HEAD = lambda self: self._authorised() and self._send(200 if urlsplit(self.path).path.rsplit("/", 1)[1] in self.blobs else 404)   # noqa: E731

    def do_POST(self):
        if self._authorised():
            self._send(202, b"", {"Location": urlsplit(self.path).path + "u1"})

    def do_PUT(self):
        n = int(self.headers.get("Content-Length") or 0)
        body = self.rfile.read(n) if n else b""
        if self.headers.get("Transfer-Encoding") == "chunked":
            body = b""
            while True:
                size = int(self.rfile.readline().strip() or b"0", 16)
                if size == 0:
                    self.rfile.readline()
                    break
                body += self.rfile.read(size)
                self.rfile.readline()
        if not self._authorised():
            return
        u = urlsplit(self.path)
        if "/manifests/" in u.path:
            self.manifests[u.path] = body
            return self._send(201)
        digest = parse_qs(u.query)["digest"][0]
        if "sha256:" + hashlib.sha256(body).hexdigest() != digest:
            return self._send(400, b"digest mismatch")
        self.blobs[digest] = body
        self._send(201)


@pytest.fixture
def registry(tmp_path, monkeypatch):
    monkeypatch.setenv("HOME", str(tmp_path / "home"))
    _Registry.blobs, _Registry.manifests, _Registry.seen = {}, {}, {"signed": [], "ranges": []}
    _Registry.pubkey_blob = auth.ensure_key().split(" ")[1]
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _Registry)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    yield f"127.0.0.1:{srv.server_address[1]}"
    srv.shutdown()


def test_push_then_pull_with_signed_token_requests(registry, tmp_path, monkeypatch):
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path / "a"))
    weights = os.urandom(300_000)
    layers = [M.new_layer(weights, M.MT_MODEL), M.new_layer(b"be brief", M.MT_SYSTEM)]
    cfg = M.new_layer(b'{"model_format":"gguf"}', M.MT_CONFIG)
    name = f"{registry}/me/thing:v1"
    M.write_manifest(parse_name(name), cfg, layers)
    st = [s["status"] for s in reg.push_model(name, insecure=True)]
    assert st[0] == "retrieving manifest" and st[-2:] == ["pushing manifest", "success"]
    assert len(_Registry.blobs) == 3 and len(_Registry.seen["signed"]) == 1          # one challenge, one signed token request, then the bearer token
    again = list(reg.push_model(name, insecure=True))                                   # everything is there already: no uploads
    assert all(s.get("completed") == s.get("total") for s in again if "digest" in s)
    # a second store pulls it; the big blob arrives through ranged requests and is verified
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path / "b"))
    monkeypatch.setattr(reg, "MIN_PART", 100_000)
    monkeypatch.setattr(reg, "MAX_PART", 100_000)
    st = list(reg.pull_model(name, insecure=True))
    assert st[0]["status"] == "pulling manifest" and st[-1]["status"] == "success"
    m = M.read_manifest(parse_name(name))
    assert m.layer(M.MT_MODEL).read() == weights and m.layer(M.MT_SYSTEM).read() == b"be brief"
    assert sorted(r for r in _Registry.seen["ranges"] if r[1] - r[0] == 99_999)[:3] == [(0, 99_999), (100_000, 199_999), (200_000, 299_999)]
    # a corrupted blob on the server is refused
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path / "c"))
    _Registry.blobs[layers[0].digest] = weights[:-1] + b"x"
    with pytest.raises(reg.RegistryError, match="digest mismatch|failed"):
        list(reg.pull_model(name, insecure=True))
    with pytest.raises(reg.RegistryError) as e:
        list(reg.pull_model(f"{registry}/me/none:v1", insecure=True))
    assert e.value.status == 404


def test_key_pair_and_challenge_url(tmp_path):
    p = str(tmp_path / "k" / "id_ed25519")
    pub = auth.ensure_key(p)
    assert pub.startswith("ssh-ed25519 ") and auth.ensure_key(p) == pub and os.stat(p).st_mode & 0o777 == 0o600       # created once
    assert open(p + ".pub").read().strip() == pub and open(p).read().startswith("-----BEGIN OPENSSH PRIVATE KEY-----")
    blob, sig = auth.sign(b"data", p).split(":")
    assert blob == pub.split(" ")[1] and len(base64.b64decode(sig)) == 64
    u = auth.challenge_url("https://r.example/token?x=1", "svc", "repository:a/b:pull repository:a/b:push", now=5, nonce="N")
    assert u == "https://r.example/token?nonce=N&scope=repository%3Aa%2Fb%3Apull&scope=repository%3Aa%2Fb%3Apush&service=svc&ts=5&x=1"
    with pytest.raises(auth.AuthError):
        auth.sign(b"x", str(tmp_path / "missing"))
    # a challenge that points at another host never gets a signature
    s = reg._Session()
    with pytest.raises(reg.RegistryError, match="does not match"):
        s._token({"realm": "http://evil.example/token", "service": "s", "scope": "x"}, "http://127.0.0.1:9/v2/a/b/manifests/t")
