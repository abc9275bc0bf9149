"""Content-addressed model store: manifests + sha256 blobs.

Same on-disk layout as the reference so an existing ``$OLLAMA_MODELS`` directory is readable:
``manifests/<host>/<namespace>/<model>/<tag>`` (JSON: schemaVersion, mediaType, config, layers;
manifest/manifest.go:16-25, manifest/layer.go:12-19) and ``blobs/sha256-<hex>``
(manifest/paths.go:17-62).  Layers are typed by media type (server/images.go:716-787).
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import shutil
import tempfile
from dataclasses import dataclass, field
from typing import Any, BinaryIO, Iterator

from .. import envconfig
from .names import Name, parse_name

MT_MANIFEST = "application/vnd.docker.distribution.manifest.v2+json"
MT_CONFIG = "application/vnd.docker.container.image.v1+json"
MT_MODEL = "application/vnd.ollama.image.model"
MT_PROJECTOR = "application/vnd.ollama.image.projector"
MT_ADAPTER = "application/vnd.ollama.image.adapter"
MT_DRAFT = "application/vnd.ollama.image.draft"
MT_TEMPLATE = "application/vnd.ollama.image.template"
MT_PROMPT = "application/vnd.ollama.image.prompt"
MT_SYSTEM = "application/vnd.ollama.image.system"
MT_PARAMS = "application/vnd.ollama.image.params"
MT_MESSAGES = "application/vnd.ollama.image.messages"
MT_LICENSE = "application/vnd.ollama.image.license"
MT_TENSOR = "application/vnd.ollama.image.tensor"
MT_JSON = "application/vnd.ollama.image.json"

_DIGEST = re.compile(r"^sha256[:-][0-9a-fA-F]{64}$")


class StoreError(Exception):
    pass


def models_root() -> str:
    return envconfig.models_dir()


def manifests_dir() -> str:
    p = os.path.join(models_root(), "manifests")
    os.makedirs(p, exist_ok=True)
    return p


def blobs_dir() -> str:
    p = os.path.join(models_root(), "blobs")
    os.makedirs(p, exist_ok=True)
    return p


def blob_path(digest: str) -> str:
    """Path of a blob; ``digest`` may be written ``sha256:<hex>`` or ``sha256-<hex>``."""
    if digest and not _DIGEST.match(digest):
        raise StoreError("invalid digest format")
    return os.path.join(blobs_dir(), digest.replace(":", "-"))


def manifest_path(name: Name) -> str:
    if not name.valid:
        raise StoreError(f"invalid model name: {name}")
    return os.path.join(manifests_dir(), *name.filepath().split("/"))


@dataclass
class Layer:
    media_type: str
    digest: str
    size: int
    from_: str = ""
    name: str = ""

    def to_json(self) -> dict[str, Any]:
        d: dict[str, Any] = {"mediaType": self.media_type, "digest": self.digest, "size": self.size}
        if self.from_:
            d["from"] = self.from_
        if self.name:
            d["name"] = self.name
        return d

    @staticmethod
    def from_json(d: dict[str, Any]) -> "Layer":
        return Layer(d.get("mediaType", ""), d.get("digest", ""), int(d.get("size", 0)), d.get("from", ""), d.get("name", ""))

    def path(self) -> str:
        return blob_path(self.digest)

    def read(self) -> bytes:
        with open(self.path(), "rb") as f:
            return f.read()


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return "sha256:" + h.hexdigest()


def new_layer(data: bytes | BinaryIO | str, media_type: str) -> Layer:
    """Store ``data`` (bytes, a readable stream, or a path to copy) as a blob and return its layer."""
    fd, tmp = tempfile.mkstemp(prefix="sha256-", dir=blobs_dir())
    h = hashlib.sha256()
    size = 0
    try:
        with os.fdopen(fd, "wb") as out:
            if isinstance(data, (bytes, bytearray)):
                out.write(data)
                h.update(data)
                size = len(data)
            else:
                src = open(data, "rb") if isinstance(data, str) else data
                try:
                    for chunk in iter(lambda: src.read(1 << 22), b""):
                        out.write(chunk)
                        h.update(chunk)
                        size += len(chunk)
                finally:
                    if isinstance(data, str):
                        src.close()
        digest = "sha256:" + h.hexdigest()
        dst = blob_path(digest)
        if os.path.exists(dst):
            os.unlink(tmp)
        else:
            os.replace(tmp, dst)
            os.chmod(dst, 0o644)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise
    return Layer(media_type, digest, size)


def layer_from_existing(digest: str, media_type: str, from_: str = "") -> Layer:
    p = blob_path(digest)
    if not os.path.exists(p):
        raise StoreError(f"blob {digest} does not exist")
    return Layer(media_type, digest.replace("-", ":", 1) if digest.startswith("sha256-") else digest, os.path.getsize(p), from_)


@dataclass
class Manifest:
    config: Layer
    layers: list[Layer] = field(default_factory=list)
    schema_version: int = 2
    media_type: str = MT_MANIFEST
    path: str = ""
    digest: str = ""
    mtime: float = 0.0

    def size(self) -> int:
        return sum(l.size for l in self.layers) + self.config.size

    def to_json(self) -> dict[str, Any]:
        return {"schemaVersion": self.schema_version, "mediaType": self.media_type, "config": self.config.to_json(),
                "layers": [l.to_json() for l in self.layers]}

    def config_json(self) -> dict[str, Any]:
        try:
            return json.loads(self.config.read())
        except (OSError, ValueError):
            return {}

    def layer(self, media_type: str) -> Layer | None:
        for l in self.layers:
            if l.media_type == media_type:
                return l
        return None


def read_manifest(name: Name) -> Manifest:
    p = manifest_path(name)
    try:
        with open(p, "rb") as f:
            raw = f.read()
    except FileNotFoundError:
        raise StoreError(f"model '{name.display()}' not found") from None
    d = json.loads(raw)
    m = Manifest(Layer.from_json(d.get("config", {})), [Layer.from_json(x) for x in d.get("layers", [])],
                 int(d.get("schemaVersion", 2)), d.get("mediaType", MT_MANIFEST), p, hashlib.sha256(raw).hexdigest(), os.path.getmtime(p))
    return m


def write_manifest(name: Name, config: Layer, layers: list[Layer]) -> Manifest:
    p = manifest_path(name)
    os.makedirs(os.path.dirname(p), exist_ok=True)
    m = Manifest(config, layers)
    tmp = p + ".tmp"
    with open(tmp, "w") as f:
        json.dump(m.to_json(), f)
    os.replace(tmp, p)
    return read_manifest(name)


def manifest_names() -> Iterator[tuple[Name, str]]:
    """Every stored model name with the path of its manifest file (nothing is read)."""
    root = manifests_dir()
    if not os.path.isdir(root):
        return
    for host in sorted(os.listdir(root)):
        hp = os.path.join(root, host)
        if not os.path.isdir(hp):
            continue
        for dirpath, _, files in os.walk(hp):
            rel = os.path.relpath(dirpath, root).split(os.sep)
            if len(rel) != 3:
                continue
            for tag in sorted(files):
                if tag.endswith(".tmp"):
                    continue
                n = Name(rel[0], rel[1], rel[2], tag)
                if n.valid:
                    yield n, os.path.join(dirpath, tag)


def list_manifests() -> Iterator[tuple[Name, Manifest]]:
    for n, _ in manifest_names():
        try:
            yield n, read_manifest(n)
        except (StoreError, ValueError, OSError):
            continue


def delete_model(name: Name) -> None:
    """Remove the manifest and those of its own blobs that no other manifest uses (manifest/manifest.go RemoveLayers).

    Blobs that belong to no manifest at all are left alone: they may be uploads waiting for a create, or the finished
    layers of a pull or create that has not written its manifest yet.  Unreferenced blobs are only swept at start-up
    (:func:`prune_layers`).  A manifest that cannot be parsed counts as using nothing, exactly as at start-up, but its
    blobs are not candidates here either, because only the deleted manifest's layers are.
    """
    m = read_manifest(name)
    os.unlink(m.path)
    mine = {m.config.digest.replace(":", "-")} | {l.digest.replace(":", "-") for l in m.layers}
    mine.discard("")
    in_use = set()
    for _, other in list_manifests():
        in_use.add(other.config.digest.replace(":", "-"))
        in_use.update(l.digest.replace(":", "-") for l in other.layers)
    for fn in mine - in_use:
        if fn.startswith("sha256-") and len(fn) == 71:
            try:
                os.unlink(os.path.join(blobs_dir(), fn))
            except FileNotFoundError:
                pass
    prune_empty_dirs(manifests_dir())


def copy_model(src: Name, dst: Name) -> None:
    sp, dp = manifest_path(src), manifest_path(dst)
    if not os.path.exists(sp):
        raise StoreError(f"model '{src.display()}' not found")
    os.makedirs(os.path.dirname(dp), exist_ok=True)
    shutil.copyfile(sp, dp)


def prune_layers() -> int:
    """Delete blobs that no manifest references; returns how many were removed."""
    used = set()
    for _, m in list_manifests():
        used.add(m.config.digest.replace(":", "-"))
        used.update(l.digest.replace(":", "-") for l in m.layers)
    n = 0
    for fn in os.listdir(blobs_dir()):
        if fn.startswith("sha256-") and fn not in used and not fn.endswith("-partial") and "-partial-" not in fn:
            if len(fn) == 71:
                os.unlink(os.path.join(blobs_dir(), fn))
                n += 1
    return n


def prune_empty_dirs(root: str) -> None:
    for dirpath, dirs, files in os.walk(root, topdown=False):
        if dirpath != root and not dirs and not files:
            try:
                os.rmdir(dirpath)
            except OSError:
                pass


def fix_blobs() -> None:
    """Older stores named blobs ``sha256:<hex>``; rename them to the portable ``sha256-<hex>``."""
    d = blobs_dir()
    for fn in os.listdir(d):
        if fn.startswith("sha256:"):
            os.replace(os.path.join(d, fn), os.path.join(d, fn.replace(":", "-", 1)))
