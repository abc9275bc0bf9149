"""Identity of this installation: an ed25519 key pair under ``~/.ollama`` and request signing for registries.

The server creates the key pair the first time it starts (cmd/cmd.go:2033-2077); ``id_ed25519`` is an OpenSSH
private key, ``id_ed25519.pub`` the matching ``ssh-ed25519 ...`` line that a user registers with a registry
account.  A registry answers a request for a private namespace with a bearer challenge; the token request
that follows carries ``Authorization: <public key blob, base64>:<signature, base64>`` where the signature
covers ``"GET,<token url>,<base64 of the hex SHA-256 of the empty body>"`` (auth/auth.go:54-90,
server/auth.go:28-75).
"""
from __future__ import annotations

import base64
import hashlib
import os
import secrets
import time
from urllib.parse import parse_qsl, urlencode, urlsplit, urlunsplit

KEY_NAME = "id_ed25519"


class AuthError(Exception):
    pass


def key_path() -> str:
    return os.path.join(os.path.expanduser("~"), ".ollama", KEY_NAME)


def _crypto():
    try:
        from cryptography.hazmat.primitives import serialization
        from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey
        return serialization, Ed25519PrivateKey
    except ImportError as e:          # the package is optional: only signing needs it
        raise AuthError(f"ed25519 support is not available: {e}") from None


def ensure_key(path: str | None = None) -> str:
    """Create the key pair unless the private key exists already; returns the public key line."""
    path = path or key_path()
    ser, Key = _crypto()
    if not os.path.exists(path):
        os.makedirs(os.path.dirname(path), mode=0o755, exist_ok=True)
        key = Key.generate()
        pem = key.private_bytes(ser.Encoding.PEM, ser.PrivateFormat.OpenSSH, ser.NoEncryption())
        fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o600)
        with os.fdopen(fd, "wb") as f:
            f.write(pem)
        pub = key.public_key().public_bytes(ser.Encoding.OpenSSH, ser.PublicFormat.OpenSSH)
        with open(path + ".pub", "wb") as f:
            f.write(pub + b"\n")
        os.chmod(path + ".pub", 0o644)
    return public_key(path)


def _load(path: str | None):
    ser, Key = _crypto()
    path = path or key_path()
    try:
        with open(path, "rb") as f:
            key = ser.load_ssh_private_key(f.read(), password=None)
    except OSError as e:
        raise AuthError(f"failed to load private key: {e}") from None
    except ValueError as e:
        raise AuthError(f"malformed private key: {e}") from None
    if not isinstance(key, Key):
        raise AuthError("the private key is not an ed25519 key")
    return ser, key


def public_key(path: str | None = None) -> str:
    """``ssh-ed25519 <base64 blob>`` of the stored key."""
    ser, key = _load(path)
    return key.public_key().public_bytes(ser.Encoding.OpenSSH, ser.PublicFormat.OpenSSH).decode().strip()


def sign(data: bytes, path: str | None = None) -> str:
    """``<public key blob>:<signature>``, both standard base64."""
    ser, key = _load(path)
    parts = key.public_key().public_bytes(ser.Encoding.OpenSSH, ser.PublicFormat.OpenSSH).split(b" ")
    if len(parts) < 2:
        raise AuthError("malformed public key")
    return f"{parts[1].strip().decode()}:{base64.b64encode(key.sign(data)).decode()}"


def new_nonce(length: int = 16) -> str:
    return base64.urlsafe_b64encode(secrets.token_bytes(length)).rstrip(b"=").decode()


def challenge_url(realm: str, service: str, scope: str, now: int | None = None, nonce: str | None = None) -> str:
    """Token URL of a bearer challenge: the realm plus service, one ``scope`` per space-separated entry, a time stamp
    and a nonce, keys in sorted order."""
    u = urlsplit(realm)
    q = parse_qsl(u.query, keep_blank_values=True)
    q.append(("service", service))
    q += [("scope", s) for s in scope.split(" ")]
    q.append(("ts", str(int(time.time()) if now is None else now)))
    q.append(("nonce", nonce or new_nonce()))
    q.sort(key=lambda kv: kv[0])          # stable: repeated keys keep their order
    return urlunsplit((u.scheme, u.netloc, u.path, urlencode(q), u.fragment))


def token_request_signature(url: str, path: str | None = None) -> str:
    empty = base64.b64encode(hashlib.sha256(b"").hexdigest().encode()).decode()
    return sign(f"GET,{url},{empty}".encode(), path)
