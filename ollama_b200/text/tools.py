"""Generic streaming tool-call extraction.

The tag that precedes tool-call JSON (``<tool_call>``, ``[TOOL_CALLS]``, ``<|python_tag|>`` ... or
just ``{``) is derived from the prompt template: it is the literal text printed right before the
template ranges over ``.ToolCalls`` (tools/template.go).  While streaming, content before the tag
passes through; after it, every balanced JSON object whose name matches a declared tool and whose
argument keys belong to that tool becomes a call (tools/tools.go:54-108, :168-347).
"""
from __future__ import annotations

import json
import random
import re
import string
from typing import Any


def tool_call_id() -> str:
    return "call_" + "".join(random.choices(string.ascii_lowercase + string.digits, k=8))


def infer_tag(template_src: str) -> str:
    """Literal text before ``{{ range .ToolCalls }}`` in a Go template (or before tool-call JSON in a Jinja one)."""
    m = re.search(r"\{\{-?\s*range\s+(?:\$\w+\s*(?:,\s*\$\w+\s*)?:=\s*)?\$?\.?ToolCalls", template_src)
    if m:
        before = template_src[:m.start()]
        lit = re.split(r"\{\{.*?\}\}", before, flags=re.S)[-1]
        lit = lit.strip()
        if lit:
            return lit.split()[-1] if " " in lit and not lit.startswith("<") else lit
        # the literal may sit inside the range body
        body = template_src[m.end():]
        body = body[body.find("}}") + 2:]
        lit = re.split(r"\{\{", body, maxsplit=1)[0].strip()
        return lit.split("{")[0].strip() or "{"
    for tag in ("<tool_call>", "[TOOL_CALLS]", "<|python_tag|>", "<|tool_call|>", "<function_call>"):
        if tag in template_src:
            return tag
    return "{"


def _find_objects(buf: str) -> tuple[list[tuple[Any, int, int]], bool]:
    """Balanced top-level JSON objects / arrays in ``buf``: [(value, start, end)], and whether one is still open."""
    out = []
    i, n = 0, len(buf)
    while i < n:
        if buf[i] not in "{[":
            i += 1
            continue
        depth, j, in_str, esc = 0, i, False, False
        while j < n:
            ch = buf[j]
            if in_str:
                if esc:
                    esc = False
                elif ch == "\\":
                    esc = True
                elif ch == '"':
                    in_str = False
            elif ch == '"':
                in_str = True
            elif ch in "{[":
                depth += 1
            elif ch in "}]":
                depth -= 1
                if depth == 0:
                    break
            j += 1
        if j >= n:
            return out, True
        try:
            out.append((json.loads(buf[i:j + 1]), i, j + 1))
        except ValueError:
            pass
        i = j + 1
    return out, False


class ToolParser:
    def __init__(self, tools: list[dict[str, Any]], tag: str = "{"):
        self.tools = {t.get("function", {}).get("name", ""): t.get("function", {}) for t in tools or []}
        self.tag = tag or "{"
        self.buf = ""
        self.in_call = False
        self.n = 0
        self.done = False

    def _hold(self, s: str) -> int:
        for k in range(min(len(self.tag), len(s)), 0, -1):
            if s.endswith(self.tag[:k]):
                return k
        return 0

    def _match(self, obj: Any) -> list[dict[str, Any]]:
        calls = []
        items = obj if isinstance(obj, list) else [obj]
        for o in items:
            if not isinstance(o, dict):
                continue
            if isinstance(o.get("function"), dict):
                o = o["function"]
            name = o.get("name") or o.get("function")
            if not isinstance(name, str) or name not in self.tools:
                continue
            args = o.get("arguments", o.get("parameters", {}))
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except ValueError:
                    continue
            if not isinstance(args, dict):
                continue
            calls.append({"id": tool_call_id(), "function": {"index": self.n, "name": name, "arguments": args}})
            self.n += 1
        return calls

    def add(self, s: str) -> tuple[list[dict[str, Any]], str]:
        """Feed model output; returns (tool calls completed now, content to show)."""
        if self.done or not self.tools:
            return [], s
        self.buf += s
        if not self.in_call:
            i = self.buf.find(self.tag)
            if i < 0:
                k = self._hold(self.buf)
                out, self.buf = self.buf[:len(self.buf) - k], self.buf[len(self.buf) - k:]
                return [], out
            # the tag must start the message or follow whitespace: prose that merely contains "{" is content
            if self.tag == "{" and self.buf[:i].strip():
                out, self.buf = self.buf, ""
                self.done = True
                return [], out
            content = self.buf[:i]
            self.buf = self.buf[i if self.tag in "{[" else i + len(self.tag):]
            self.in_call = True
        else:
            content = ""
        objs, open_ = _find_objects(self.buf)
        calls: list[dict[str, Any]] = []
        end = 0
        for obj, _, e in objs:
            got = self._match(obj)
            calls += got
            end = e
        if objs and not calls and not open_:
            # JSON that is not a call to a known tool: give it back as content
            out, self.buf = self.buf, ""
            self.in_call = False
            self.done = True
            return [], content + out
        if end:
            self.buf = self.buf[end:]
        return calls, content        # text before the tag is passed on unchanged (tools/tools_test.go "text before tool call")

    def flush(self) -> str:
        out, self.buf = self.buf, ""
        return "" if self.in_call and self.n else out
