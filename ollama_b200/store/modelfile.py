"""Modelfile parser and serialiser.

Commands ``FROM LICENSE TEMPLATE SYSTEM ADAPTER DRAFT RENDERER PARSER PARAMETER MESSAGE REQUIRES``
(case-insensitive), ``#`` comments, values either to the end of the line, ``"quoted"`` or
``\"\"\"multi-line\"\"\"`` -- the grammar of the reference's rune state machine
(parser/parser.go:425-642, quoting :644-675, command list :697-704) -- and the translation of a
parsed file into a create request (parser/parser.go:56-183).
"""
from __future__ import annotations

import shlex
from dataclasses import dataclass, field
from typing import Any

from ..api.types import DEPRECATED_PARAMETERS, format_parameters

COMMANDS = ("from", "license", "template", "system", "adapter", "draft", "renderer", "parser", "parameter", "message", "requires")
ROLES = ("system", "user", "assistant")


class ModelfileError(ValueError):
    pass


@dataclass
class Command:
    name: str          # lower-case command; for PARAMETER the parameter name
    args: str
    is_parameter: bool = False

    def __str__(self) -> str:
        if self.is_parameter:
            return f"PARAMETER {self.name} {_quote(self.args)}"
        if self.name == "from":
            return f"FROM {self.args}"
        if self.name == "message":
            role, _, content = self.args.partition(": ")
            return f"MESSAGE {role} {_quote(content)}"
        return f"{self.name.upper()} {_quote(self.args)}"


@dataclass
class Modelfile:
    commands: list[Command] = field(default_factory=list)

    def __str__(self) -> str:
        return "\n".join(str(c) for c in self.commands) + "\n"

    def get(self, name: str) -> list[str]:
        return [c.args for c in self.commands if c.name == name and not c.is_parameter]

    def create_request(self) -> dict[str, Any]:
        """Fields of an ``/api/create`` body (file paths are left for the client to hash and upload)."""
        req: dict[str, Any] = {}
        params: dict[str, list[str]] = {}
        messages, licenses = [], []
        for c in self.commands:
            if c.is_parameter:
                params.setdefault(c.name, []).append(c.args)
            elif c.name == "from":
                req["from"] = c.args
            elif c.name == "adapter":
                req.setdefault("adapter_paths", []).append(c.args)
            elif c.name == "draft":
                req.setdefault("draft_paths", []).append(c.args)
            elif c.name in ("template", "system", "renderer", "parser", "requires"):
                req[c.name] = c.args
            elif c.name == "license":
                licenses.append(c.args)
            elif c.name == "message":
                role, _, content = c.args.partition(": ")
                messages.append({"role": role, "content": content})
        if params:
            req["parameters"] = format_parameters(params)
        if messages:
            req["messages"] = messages
        if licenses:
            req["license"] = licenses
        return req


def _quote(s: str) -> str:
    if "\n" in s or '"' in s:
        return f'"""{s}"""'
    if s != s.strip() or s == "":
        return f'"{s}"'
    return s


def _unquote(s: str) -> tuple[str, bool]:
    """Value of a (possibly quoted) buffer and whether its quotes are closed (parser/parser.go:656-675)."""
    if s.startswith('"""'):
        return (s[3:-3], True) if len(s) >= 6 and s.endswith('"""') else ("", False)
    if s.startswith('"'):
        return (s[1:-1], True) if len(s) >= 2 and s.endswith('"') else ("", False)
    return s, True


def _take_value(text: str, i: int) -> tuple[str, int]:
    """Read one value starting at ``i``: the rest of the line, or, when it opens with ``"`` or ``\"\"\"``, every line
    up to the first one that ends with the closing quotes (so quotes inside a line never end the value)."""
    n = len(text)
    j = i
    while True:
        k = text.find("\n", j)
        val, ok = _unquote(text[i:(n if k < 0 else k)].strip())
        if ok:
            return val, (n if k < 0 else k + 1)
        if k < 0:
            raise ModelfileError("unexpected EOF: unterminated quoted value")
        j = k + 1


def decode_modelfile(data: bytes) -> str:
    """Text of a Modelfile: UTF-8 unless a byte-order mark says UTF-16, as the reference's BOM-overriding
    reader does (parser/parser.go:462-463)."""
    if data[:2] in (b"\xff\xfe", b"\xfe\xff"):
        return data.decode("utf-16")
    return data.decode("utf-8-sig", "replace")


def parse_modelfile(text: str | bytes) -> Modelfile:
    if isinstance(text, (bytes, bytearray)):
        text = decode_modelfile(bytes(text))
    text = text.replace("\r\n", "\n")
    if text.startswith("\ufeff"):
        text = text[1:]
    mf = Modelfile()
    i, n = 0, len(text)
    while i < n:
        # skip blank lines and comments
        j = i
        while j < n and text[j] in " \t":
            j += 1
        if j >= n:
            break
        if text[j] == "\n":
            i = j + 1
            continue
        if text[j] == "#":
            k = text.find("\n", j)
            i = n if k < 0 else k + 1
            continue
        k = j
        while k < n and not text[k].isspace():
            k += 1
        word = text[j:k].lower()
        if word not in COMMANDS:
            names = ", ".join(f'"{c}"' for c in COMMANDS[:-1]) + f', or "{COMMANDS[-1]}"'
            raise ModelfileError(f"command must be one of {names}")
        if word == "parameter":
            while k < n and text[k] in " \t":
                k += 1
            e = k
            while e < n and not text[e].isspace():
                e += 1
            pname = text[k:e].lower()
            if not pname or e >= n or text[e] == "\n":
                raise ModelfileError("unexpected EOF: PARAMETER needs a name and a value")
            val, i = _take_value(text, e)
            if pname not in DEPRECATED_PARAMETERS or True:
                mf.commands.append(Command(pname, val, True))
        elif word == "message":
            while k < n and text[k] in " \t":
                k += 1
            e = k
            while e < n and not text[e].isspace():
                e += 1
            role = text[k:e].lower()
            if role not in ROLES:
                raise ModelfileError('message role must be one of "system", "user", or "assistant"')
            if e >= n or text[e] == "\n":
                raise ModelfileError("unexpected EOF: MESSAGE needs a role and a text")
            val, i = _take_value(text, e)
            mf.commands.append(Command("message", f"{role}: {val}"))
        else:
            val, i = _take_value(text, k)
            mf.commands.append(Command(word, val))
    if not mf.get("from"):
        raise ModelfileError("no FROM line")
    return mf
