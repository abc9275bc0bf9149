"""Model names: ``[host/][namespace/]model[:tag]`` with the defaults registry.ollama.ai / library / latest.

Grammar, defaults and the on-disk path of a name follow types/model/name.go:93-300 of the reference.
"""
from __future__ import annotations

import re
from dataclasses import dataclass

DEFAULT_HOST = "registry.ollama.ai"
DEFAULT_NAMESPACE = "library"
DEFAULT_TAG = "latest"

_HOST = re.compile(r"^[A-Za-z0-9_][A-Za-z0-9_.:\-]{0,349}$")
_NAMESPACE = re.compile(r"^[A-Za-z0-9_][A-Za-z0-9_\-]{0,79}$")
_MODEL = re.compile(r"^[A-Za-z0-9_][A-Za-z0-9_.\-]{0,79}$")
_TAG = re.compile(r"^[A-Za-z0-9_][A-Za-z0-9_.\-]{0,79}$")


class InvalidName(ValueError):
    pass


@dataclass(frozen=True)
class Name:
    host: str = ""
    namespace: str = ""
    model: str = ""
    tag: str = ""

    @property
    def valid(self) -> bool:
        return bool(_HOST.match(self.host) and _NAMESPACE.match(self.namespace) and _MODEL.match(self.model) and _TAG.match(self.tag))

    def __str__(self) -> str:
        return f"{self.host}/{self.namespace}/{self.model}:{self.tag}"

    def display(self) -> str:
        """Shortest unambiguous form: default host / namespace are dropped (what `list` prints)."""
        s = self.model
        if self.namespace != DEFAULT_NAMESPACE or self.host != DEFAULT_HOST:
            s = f"{self.namespace}/{s}"
        if self.host != DEFAULT_HOST:
            s = f"{self.host}/{s}"
        return f"{s}:{self.tag}"

    def filepath(self) -> str:
        return "/".join((self.host, self.namespace, self.model, self.tag))

    def with_tag(self, tag: str) -> "Name":
        return Name(self.host, self.namespace, self.model, tag)


def parse_name(s: str, fill_defaults: bool = True) -> Name:
    """Split from the right: tag after the last ':' (unless it is a port), then model, namespace, host."""
    s = s.strip()
    scheme = re.match(r"^[a-z]+://", s)
    if scheme:
        s = s[scheme.end():]
    if "@" in s:                      # digests are not addressable here
        s = s.split("@", 1)[0]
    tag = ""
    i = s.rfind(":")
    if i >= 0 and "/" not in s[i:]:
        s, tag = s[:i], s[i + 1:]
    parts = s.split("/")
    if len(parts) > 3:
        host, namespace, model = "/".join(parts[:-2]), parts[-2], parts[-1]
    elif len(parts) == 3:
        host, namespace, model = parts
    elif len(parts) == 2:
        host, (namespace, model) = "", parts
    else:
        host, namespace, model = "", "", parts[0]
    if fill_defaults:
        host, namespace, tag = host or DEFAULT_HOST, namespace or DEFAULT_NAMESPACE, tag or DEFAULT_TAG
    return Name(host, namespace, model, tag)


def require_valid(s: str) -> Name:
    n = parse_name(s)
    if not n.valid:
        raise InvalidName(f"invalid model name: {s!r}")
    return n
