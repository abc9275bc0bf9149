"""Prompt templates: Modelfile Go templates and GGUF Jinja chat templates.

``Template`` reproduces the execution modes of the reference (template/template.go:257-350):
suffix / fill-in-the-middle, a ``.Messages`` loop, and the legacy per-turn mode in which the
template is run once per (system, user, assistant) turn and the final run is cut right where
``.Response`` starts.  A template that references neither ``.Messages`` nor ``.Response`` gets
``{{ .Response }}`` appended (:145-165).  Consecutive messages of one role are merged and every
system message also feeds ``.System`` (:357-374).

``JinjaChatTemplate`` renders ``tokenizer.chat_template`` (which the reference hands to its engine
process) in a sandbox with the ``enable_thinking`` / ``reasoning_effort`` kwargs
(llm/llama_server.go:2189-2203).
"""
from __future__ import annotations

import datetime
import json
from typing import Any

from .gotemplate import GoTemplate, TemplateError

_SENTINEL = "\x00<response>\x00"
DEFAULT_TEMPLATE = "{{ .Prompt }}"


def collate(messages: list[dict[str, Any]]) -> tuple[str, list[dict[str, Any]]]:
    system: list[str] = []
    out: list[dict[str, Any]] = []
    for m in messages:
        role = m.get("role", "")
        if role == "system":
            system.append(m.get("content", ""))
        if out and out[-1].get("role") == role and role != "tool":
            out[-1]["content"] = out[-1].get("content", "") + "\n\n" + m.get("content", "")
        else:
            out.append(dict(m))
    return "\n\n".join(system), out


def _tmpl_message(m: dict[str, Any]) -> dict[str, Any]:
    calls = []
    for tc in m.get("tool_calls") or []:
        fn = tc.get("function", {})
        calls.append({"ID": tc.get("id", ""), "Function": {"Index": fn.get("index", 0), "Name": fn.get("name", ""),
                                                           "Arguments": _Args(fn.get("arguments") or {})}})
    return {"Role": m.get("role", ""), "Content": m.get("content", ""), "Thinking": m.get("thinking", ""), "Images": m.get("images") or [],
            "ToolCalls": calls, "ToolName": m.get("tool_name", ""), "ToolCallID": m.get("tool_call_id", "")}


class _Args(dict):
    """Tool-call arguments: a map that prints as JSON inside templates."""

    def __str__(self) -> str:
        return json.dumps(self, separators=(",", ":"), ensure_ascii=False)


class _Tool(dict):
    """One tool: Go field names for templates, the wire form when printed."""

    wire: dict[str, Any] = {}

    def __str__(self) -> str:
        return json.dumps(self.wire, separators=(",", ":"), ensure_ascii=False)


_TS_TYPES = {"string": "string", "number": "number", "integer": "number", "boolean": "boolean", "array": "any[]",
             "object": "Record<string, any>", "null": "null"}


class _Prop(dict):
    """One property of a tool's parameters: the wire keys, the nested properties as :class:`_Props`, and the TypeScript
    spelling of its type that some templates ask for (api/types.go:429-471 of the reference)."""

    def __init__(self, wire: dict[str, Any]):
        super().__init__(wire)
        if isinstance(wire.get("properties"), dict):
            self["properties"] = _Props(wire["properties"])
        if isinstance(wire.get("items"), dict):
            self["items"] = _Prop(wire["items"])
        if isinstance(wire.get("anyOf"), list):
            self["anyOf"] = [_Prop(x) if isinstance(x, dict) else x for x in wire["anyOf"]]

    def ToTypeScriptType(self) -> str:      # noqa: N802 -- the name templates use
        if self.get("anyOf"):
            return " | ".join(x.ToTypeScriptType() for x in self["anyOf"] if isinstance(x, _Prop))
        t = self.get("type")
        types = [t] if isinstance(t, str) else [x for x in t if isinstance(x, str)] if isinstance(t, list) else []
        return " | ".join(_TS_TYPES.get(t, "any") for t in types) if types else "any"


class _Props(dict):
    """The properties of a tool's parameters: values are :class:`_Prop`; prints as JSON (template/template.go:396-404)."""

    def __init__(self, wire: dict[str, Any]):
        super().__init__({k: _Prop(v) if isinstance(v, dict) else v for k, v in wire.items()})
        self.wire = wire

    def __str__(self) -> str:
        return json.dumps(self.wire, separators=(",", ":"), ensure_ascii=False)


class _Tools(list):
    def __str__(self) -> str:
        return json.dumps([t.wire for t in self], separators=(",", ":"), ensure_ascii=False)


def _tmpl_tools(tools: list[dict[str, Any]] | None) -> _Tools:
    out = _Tools()
    for t in tools or []:
        fn = t.get("function", {})
        params = dict(fn.get("parameters") or {})
        if isinstance(params.get("properties"), dict):
            params["properties"] = _Props(params["properties"])
        d = _Tool({"Type": t.get("type", "function"), "Function": {"Name": fn.get("name", ""), "Description": fn.get("description", ""),
                                                                  "Parameters": params}})
        d.wire = t
        out.append(d)
    return out


class Template:
    def __init__(self, src: str):
        self.raw = src
        self.t = GoTemplate(src)
        self.vars = sorted(self.t.identifiers())
        if "messages" not in self.vars and "response" not in self.vars:
            self.t = GoTemplate(src + "{{ .Response }}")
            self.vars = sorted(self.t.identifiers())

    def __str__(self) -> str:
        return self.raw

    def contains(self, *needles: str) -> bool:
        return any(n in self.raw for n in needles)

    def execute(self, *, messages: list[dict[str, Any]] | None = None, tools: list[dict[str, Any]] | None = None, prompt: str = "",
                suffix: str = "", think: bool = False, think_level: str = "", is_think_set: bool = False,
                force_legacy: bool = False, response: str = "") -> str:
        base = {"Think": think, "ThinkLevel": think_level, "IsThinkSet": is_think_set}
        system, msgs = collate(messages or [])
        if prompt and suffix:
            return self.t.render({"Prompt": prompt, "Suffix": suffix, "Response": "", **base})
        if not force_legacy and "messages" in self.vars:
            return self.t.render({"System": system, "Messages": [_tmpl_message(m) for m in msgs], "Tools": _tmpl_tools(tools),
                                  "Response": "", **base})
        out: list[str] = []
        sys_, prm, rsp = "", "", ""

        def flush():
            nonlocal sys_, prm, rsp
            out.append(self.t.render({"System": sys_, "Prompt": prm, "Response": rsp, **base}))
            sys_, prm, rsp = "", "", ""

        for m in msgs:
            role = m.get("role")
            if role == "system":
                if prm or rsp:
                    flush()
                sys_ = m.get("content", "")
            elif role == "user":
                if rsp:
                    flush()
                prm = m.get("content", "")
            elif role == "assistant":
                rsp = m.get("content", "")
        # last run: everything after the response field is dropped so generation continues from there
        last = self.t.render({"System": sys_, "Prompt": prm, "Response": _SENTINEL, **base})
        cut = last.find(_SENTINEL)
        out.append((last[:cut] + rsp) if cut >= 0 else last)
        return "".join(out)

    def render_generate(self, system: str, prompt: str, **kw) -> str:
        """``/api/generate`` form: one system + one user turn."""
        msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": prompt}]
        return self.execute(messages=msgs, **kw)


# -- Jinja chat templates ---------------------------------------------------------------------------------
class JinjaChatTemplate:
    def __init__(self, src: str, bos_token: str = "", eos_token: str = ""):
        from jinja2 import StrictUndefined  # noqa: F401
        from jinja2.sandbox import ImmutableSandboxedEnvironment
        self.raw = src
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])

        def raise_exception(msg):
            raise TemplateError(msg)

        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        env.filters["tojson"] = lambda v, indent=None, **kw: json.dumps(v, ensure_ascii=False, indent=indent)
        try:
            self.t = env.from_string(src)
        except Exception as e:          # jinja2.TemplateSyntaxError and friends
            raise TemplateError(f"chat template: {e}") from None
        self.bos_token, self.eos_token = bos_token, eos_token

    def render(self, messages: list[dict[str, Any]], tools: list[dict[str, Any]] | None = None, add_generation_prompt: bool = True,
               **kwargs: Any) -> str:
        msgs = []
        for m in messages:
            d = {"role": m.get("role", ""), "content": m.get("content", "")}
            if m.get("tool_calls"):
                d["tool_calls"] = [{"type": "function", "id": tc.get("id", ""),
                                    "function": {"name": tc.get("function", {}).get("name", ""),
                                                 "arguments": tc.get("function", {}).get("arguments") or {}}} for tc in m["tool_calls"]]
            if m.get("thinking"):
                d["reasoning_content"] = m["thinking"]
            if m.get("tool_name"):
                d["name"] = m["tool_name"]
            if m.get("tool_call_id"):
                d["tool_call_id"] = m["tool_call_id"]
            msgs.append(d)
        try:
            return self.t.render(messages=msgs, tools=tools or None, add_generation_prompt=add_generation_prompt,
                                 bos_token=self.bos_token, eos_token=self.eos_token, **kwargs)
        except TemplateError:
            raise
        except Exception as e:          # undefined names, operations on the wrong kind of value, sandbox violations
            raise TemplateError(f"chat template: {type(e).__name__}: {e}") from None


# Named templates recognised from a GGUF chat template (the reference matches against its catalogue by edit
# distance, template/template.go:72-92); the handful below covers the families served here.
NAMED_TEMPLATES = {
    "chatml": "{{- range .Messages }}<|im_start|>{{ .Role }}\n{{ .Content }}<|im_end|>\n{{ end }}<|im_start|>assistant\n",
    "llama3-instruct": "{{- range .Messages }}<|start_header_id|>{{ .Role }}<|end_header_id|>\n\n{{ .Content }}<|eot_id|>{{ end }}"
                       "<|start_header_id|>assistant<|end_header_id|>\n\n",
    "gemma-instruct": "{{- range .Messages }}<start_of_turn>{{ if eq .Role \"assistant\" }}model{{ else }}{{ .Role }}{{ end }}\n"
                      "{{ .Content }}<end_of_turn>\n{{ end }}<start_of_turn>model\n",
    "mistral-instruct": "{{- range .Messages }}{{ if eq .Role \"user\" }}[INST] {{ .Content }} [/INST]{{ else }}{{ .Content }}</s>{{ end }}{{ end }}",
    "alpaca": "{{ if .System }}{{ .System }}\n\n{{ end }}{{ if .Prompt }}### Instruction:\n{{ .Prompt }}\n\n{{ end }}### Response:\n{{ .Response }}\n\n",
}


def detect_named_template(chat_template: str) -> str | None:
    s = chat_template
    if "<|im_start|>" in s:
        return "chatml"
    if "<|start_header_id|>" in s:
        return "llama3-instruct"
    if "<start_of_turn>" in s:
        return "gemma-instruct"
    if "[INST]" in s:
        return "mistral-instruct"
    if "### Instruction" in s:
        return "alpaca"
    return None
