"""Harmony (gpt-oss) message format: streaming output parser and prompt renderer.

Wire format: ``<|start|>{role}[ to={recipient}][<|channel|>{analysis|commentary|final}[ to=functions.NAME]
[ <|constrain|>json]]<|message|>{body}<|end|>``; an assistant turn ends with ``<|return|>`` or, for a
tool call, ``<|call|>``.  Routing while streaming: ``analysis`` -> thinking, ``final`` -> content, any
header with a ``functions.*`` recipient -> tool call whose JSON body is collected until the message
ends.  The generation prompt already ends with ``<|start|>assistant``, so the parser starts inside a
header.  Tool names that are not valid identifiers are mangled on the way in and mapped back on the
way out.  Behavioural reference: harmony/harmonyparser.go:36-110 (tags, implicit start), :265-340
(header parsing), :379-556 (routing and name mapping).
"""
from __future__ import annotations

import datetime
import json
import re
from typing import Any

from .tools import tool_call_id

TAGS = ("<|start|>", "<|channel|>", "<|message|>", "<|end|>", "<|return|>", "<|call|>", "<|constrain|>")
_ANY_TAG = re.compile("|".join(re.escape(t) for t in TAGS))
HEADER, BODY, BETWEEN = range(3)


_BUILTIN_TOOLS = ("browser.open", "browser.search", "browser.find", "python")


class FunctionNameMap:
    """user tool name <-> identifier-safe harmony name (harmony/harmonyparser.go:476-556).

    Spaces, hyphens and periods become underscores; letters, digits (Unicode categories L* and Nd), ``_`` and ``$`` stay;
    everything else is dropped; an empty result is ``unnamed``; a leading digit gets an underscore in front; a name that
    is taken gets ``_2``, ``_3`` ...; the built-in tool names are kept as they are.
    """

    def __init__(self):
        self.to_h: dict[str, str] = {}
        self.from_h: dict[str, str] = {}

    @staticmethod
    def valid_chars(name: str) -> str:
        import unicodedata
        out = []
        for ch in name:
            if ch in " -.":
                out.append("_")
            elif ch in "_$" or unicodedata.category(ch)[0] == "L" or unicodedata.category(ch) == "Nd":
                out.append(ch)
        h = "".join(out) or "unnamed"
        return "_" + h if h[0] in "0123456789" else h

    def add(self, name: str) -> str:
        """A new harmony name for ``name``, even when the same user name was added before (duplicate tool definitions)."""
        base = self.valid_chars(name)
        h, k = base, 2
        while h in self.from_h:
            h = f"{base}_{k}"
            k += 1
        if name in _BUILTIN_TOOLS:
            h = name
        self.to_h[name], self.from_h[h] = h, name
        return h

    def convert(self, name: str) -> str:
        """The harmony name of ``name``: the one it already has, else a new one."""
        return self.to_h[name] if name in self.to_h else self.add(name)

    def original(self, h: str) -> str:
        return self.from_h.get(h, h)


class HarmonyParser:
    def __init__(self, names: FunctionNameMap | None = None, prefill: str = ""):
        self.names = names or FunctionNameMap()
        self.state = HEADER           # the prompt ends with "<|start|>assistant": we are inside that header
        self.header = "assistant" + prefill
        self.buf = ""
        self.channel = ""
        self.recipient = ""
        self.tool_buf = ""
        self.tool_calls: list[dict[str, Any]] = []
        self._n = 0

    def _hold(self, s: str) -> int:
        """Length of a suffix of ``s`` that could be the start of a tag."""
        for k in range(min(12, len(s)), 0, -1):
            tail = s[-k:]
            if any(t.startswith(tail) for t in TAGS):
                return k
        return 0

    def _parse_header(self, h: str) -> None:
        self.channel, self.recipient = "", ""
        h = h.replace("<|constrain|>", " <|constrain|>")
        role_part, _, chan_part = h.partition("<|channel|>")
        m = re.search(r"\bto=([^\s<]+)", role_part)
        if m:
            self.recipient = m.group(1)
        if chan_part:
            toks = chan_part.split()
            if toks:
                self.channel = toks[0]
            m = re.search(r"\bto=([^\s<]+)", chan_part)
            if m:
                self.recipient = m.group(1)

    def _finish_message(self) -> None:
        if self.recipient.startswith("functions."):
            name = self.names.original(self.recipient[len("functions."):])
            raw = self.tool_buf.strip()
            try:
                args = json.loads(raw) if raw else {}
            except ValueError:
                args = {"_raw": raw}
            if not isinstance(args, dict):
                args = {"value": args}
            self.tool_calls.append({"id": tool_call_id(), "function": {"index": self._n, "name": name, "arguments": args}})
            self._n += 1
        self.tool_buf = ""

    def add(self, s: str) -> tuple[str, str, list[dict[str, Any]]]:
        """Feed output text (special tokens rendered as text); returns (thinking, content, tool calls finished now)."""
        self.buf += s
        thinking, content = [], []
        done_before = len(self.tool_calls)
        while self.buf:
            m = _ANY_TAG.search(self.buf)
            if self.state == BODY:
                text = self.buf[:m.start()] if m else self.buf
                if not m:
                    k = self._hold(text)
                    text, self.buf = text[:len(text) - k], text[len(text) - k:]
                if text:
                    if self.recipient.startswith("functions."):
                        self.tool_buf += text
                    elif self.channel == "analysis":
                        thinking.append(text)
                    elif self.channel in ("final", ""):
                        content.append(text)
                    else:               # commentary without a recipient: preamble shown to the user
                        content.append(text)
                if not m:
                    break
                tag = m.group(0)
                self.buf = self.buf[m.end():]
                if tag in ("<|end|>", "<|return|>", "<|call|>"):
                    self._finish_message()
                    self.state = BETWEEN
                elif tag == "<|start|>":
                    self._finish_message()
                    self.state, self.header = HEADER, ""
                continue
            if self.state == BETWEEN:
                if not m:
                    k = self._hold(self.buf)
                    self.buf = self.buf[len(self.buf) - k:] if k else ""
                    break
                self.buf = self.buf[m.end():]
                if m.group(0) == "<|start|>":
                    self.state, self.header = HEADER, ""
                continue
            # HEADER: collect until <|message|>
            i = self.buf.find("<|message|>")
            if i < 0:
                k = self._hold(self.buf)
                self.header += self.buf[:len(self.buf) - k]
                self.buf = self.buf[len(self.buf) - k:]
                break
            self.header += self.buf[:i]
            self.buf = self.buf[i + len("<|message|>"):]
            self._parse_header(self.header)
            self.state = BODY
        return "".join(thinking), "".join(content), self.tool_calls[done_before:]


# ---------------------------------------------------------------------------------------------
# prompt rendering
# ---------------------------------------------------------------------------------------------
def _ts_type(schema: Any) -> str:
    if not isinstance(schema, dict):
        return "any"
    t = schema.get("type")
    if schema.get("enum"):
        return " | ".join(json.dumps(e) for e in schema["enum"])
    if isinstance(t, list):
        return " | ".join(_ts_type({**schema, "type": x}) for x in t)
    if t == "array":
        return _ts_type(schema.get("items")) + "[]"
    if t == "object":
        props = schema.get("properties") or {}
        if not props:
            return "object"
        req = set(schema.get("required") or [])
        inner = ", ".join(f"{k}{'' if k in req else '?'}: {_ts_type(v)}" for k, v in props.items())
        return "{ " + inner + " }"
    return {"string": "string", "number": "number", "integer": "number", "boolean": "boolean", "null": "null"}.get(t, "any")


def render_tools(tools: list[dict[str, Any]], names: FunctionNameMap) -> str:
    lines = ["# Tools", "", "## functions", "", "namespace functions {", ""]
    for t in tools:
        fn = t.get("function", {})
        if fn.get("description"):
            lines.append(f"// {fn['description']}")
        params = fn.get("parameters") or {}
        props = params.get("properties") or {}
        name = names.convert(fn.get("name", ""))
        if props:
            req = set(params.get("required") or [])
            lines.append(f"type {name} = (_: {{")
            for k, v in props.items():
                if isinstance(v, dict) and v.get("description"):
                    lines.append(f"// {v['description']}")
                lines.append(f"{k}{'' if k in req else '?'}: {_ts_type(v)},")
            lines.append("}) => any;")
        else:
            lines.append(f"type {name} = () => any;")
        lines.append("")
    lines.append("} // namespace functions")
    return "\n".join(lines)


def render_prompt(messages: list[dict[str, Any]], tools: list[dict[str, Any]] | None = None, think: str | bool | None = None,
                  names: FunctionNameMap | None = None, today: str | None = None) -> str:
    """Build the full harmony prompt, ending with ``<|start|>assistant``."""
    names = names or FunctionNameMap()
    level = think if isinstance(think, str) else ("medium" if think in (None, True) else "low")
    if level == "max":
        level = "high"
    today = today or datetime.date.today().isoformat()
    out = ["<|start|>system<|message|>You are ChatGPT, a large language model trained by OpenAI.\nKnowledge cutoff: 2024-06\n"
           f"Current date: {today}\n\nReasoning: {level}\n\n# Valid channels: analysis, commentary, final. Channel must be included for every message."]
    if tools:
        out.append("\nCalls to these tools must go to the commentary channel: 'functions'.")
    out.append("<|end|>")
    system = "\n\n".join(m.get("content", "") for m in messages if m.get("role") == "system")
    if system or tools:
        dev = []
        if system:
            dev.append("# Instructions\n\n" + system)
        if tools:
            dev.append(render_tools(tools, names))
        out.append("<|start|>developer<|message|>" + "\n\n".join(dev) + "<|end|>")
    last_user = max((i for i, m in enumerate(messages) if m.get("role") == "user"), default=-1)
    for i, m in enumerate(messages):
        role = m.get("role")
        if role == "user":
            out.append(f"<|start|>user<|message|>{m.get('content', '')}<|end|>")
        elif role == "assistant":
            if m.get("thinking") and i > last_user:      # reasoning of earlier turns is dropped
                out.append(f"<|start|>assistant<|channel|>analysis<|message|>{m['thinking']}<|end|>")
            for tc in m.get("tool_calls") or []:
                fn = tc.get("function", {})
                args = json.dumps(fn.get("arguments") or {}, separators=(",", ":"), ensure_ascii=False)
                out.append(f"<|start|>assistant<|channel|>commentary to=functions.{names.convert(fn.get('name', ''))} "
                           f"<|constrain|>json<|message|>{args}<|call|>")
            if m.get("content"):
                out.append(f"<|start|>assistant<|channel|>final<|message|>{m['content']}<|end|>")
        elif role == "tool":
            name = names.convert(m.get("tool_name", "") or "tool")
            out.append(f"<|start|>functions.{name} to=assistant<|channel|>commentary<|message|>{m.get('content', '')}<|end|>")
    out.append("<|start|>assistant")
    return "".join(out)
