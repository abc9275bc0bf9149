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


def _take_value(text: str, i: int) -> tuple[str, int]:
    """Read one value starting at ``i`` (after leading blanks): triple-quoted, quoted, or to end of line."""
    n = len(text)
    while i < n and text[i] in " \t":
        i += 1
    if text.startswith('"""', i):
        j = text.find('"""', i + 3)
        if j < 0:
            raise ModelfileError("unterminated multiline string")
        val = text[i + 3:j]
        k = text.find("\n", j + 3)
        return val, (n if k < 0 else k + 1)
    if i < n and text[i] == '"':
        j = i + 1
        while j < n and text[j] != '"' and text[j] != "\n":
            j += 1
        if j < n and text[j] == '"':
            k = text.find("\n", j + 1)
            return text[i + 1:j], (n if k < 0 else k + 1)
    k = text.find("\n", i)
    end = n if k < 0 else k
    return text[i:end].rstrip(" \t\r"), (n if k < 0 else k + 1)


def parse_modelfile(text: str) -> Modelfile:
    text = text.replace("\r\n", "\n")
    if text.startswith("﻿"):
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
            if not pname:
                raise ModelfileError("missing parameter name")
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
            val, i = _take_value(text, e)
            mf.commands.append(Command("message", f"{role}: {val}"))
        else:
            val, i = _take_value(text, k)
            mf.commands.append(Command(word, val))
    if not mf.get("from"):
        raise ModelfileError("no FROM line")
    return mf
