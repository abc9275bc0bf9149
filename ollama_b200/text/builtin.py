"""Built-in prompt renderers and output parsers selected by a model's ``renderer`` / ``parser`` configuration
(Modelfile RENDERER / PARSER), for model families whose chat format is not expressed by a template.

The reference keeps one Go type per family (model/renderers/renderer.go:60-120, model/parsers/parsers.go:46-110).
Here all parsers are instances of one streaming state machine over literal tags (:class:`TagStreamParser`)
that differ in their tags and in how the body of a tool call is decoded:

===================  ==========================  ===================================================================
name                 reasoning block             tool call
===================  ==========================  ===================================================================
``qwen3``            none                        ``<tool_call>{"name": .., "arguments": {..}}</tool_call>``
``qwen3-thinking``   starts inside ``<think>``   same
``qwen3-coder``      none                        ``<tool_call><function=f><parameter=k>\\nv\\n</parameter></function></tool_call>``
``ministral``        ``[THINK]..[/THINK]``       ``[TOOL_CALLS]name[ARGS]{json}``
``functiongemma``    none                        ``<start_function_call>call:name{k:<escape>v<escape>}<end_function_call>``
``passthrough``      none                        none
===================  ==========================  ===================================================================

``harmony`` is handled by :mod:`ollama_b200.text.harmony`.  Renderers: ``qwen3-coder``, ``functiongemma``.
"""
from __future__ import annotations

import json
import re
from typing import Any, Callable


# ---------------------------------------------------------------------------------------------------
# streaming parser
# ---------------------------------------------------------------------------------------------------
def _overlap(s: str, tag: str) -> int:
    """Length of the longest suffix of ``s`` that is a proper prefix of ``tag``."""
    for n in range(min(len(s), len(tag) - 1), 0, -1):
        if s.endswith(tag[:n]):
            return n
    return 0


class TagStreamParser:
    """Splits a streamed completion into content, reasoning and tool calls.

    ``add(text, done)`` returns ``(content, thinking, calls)`` for what became unambiguous with this chunk: text that
    could still turn out to be the beginning of a tag (and the white space in front of it) is held back until the
    next chunk decides, and everything held is released when ``done`` is true.
    """

    def __init__(self, *, think_open: str = "", think_close: str = "", start_thinking: bool = False, tool_open: str = "",
                 tool_close: str | None = "", decode_call: Callable[[str], dict[str, Any] | None] | None = None,
                 body_end: Callable[[str], int] | None = None):
        self.think_open, self.think_close = think_open, think_close
        self.tool_open, self.tool_close = tool_open, tool_close
        self.decode_call, self.body_end = decode_call, body_end
        self.state = "thinking" if start_thinking and think_close else "content"
        self.may_open_think = bool(think_open)        # an explicit opening tag is accepted at the very start only
        self.skip_ws = False                          # white space right after a closed block belongs to the markup
        self.buf = ""

    def add(self, text: str, done: bool = False) -> tuple[str, str, list[dict[str, Any]]]:
        self.buf += text
        content, thinking, calls = [], [], []
        while True:
            if self.state == "thinking":
                if self.may_open_think:             # some checkpoints repeat the opening tag although the prompt ended with it
                    t = self.buf.lstrip()
                    if t.startswith(self.think_open):
                        self.buf = t[len(self.think_open):]
                        self.may_open_think = False
                        continue
                    if t and not self.think_open.startswith(t):
                        self.may_open_think = False
                    elif not done:
                        break
                i = self.buf.find(self.think_close)
                if i >= 0:
                    thinking.append(self.buf[:i].rstrip())
                    self.buf = self.buf[i + len(self.think_close):]
                    self.state, self.skip_ws = "content", True
                    continue
                keep = 0 if done else self._held(self.buf, [self.think_close])
                thinking.append(self.buf[:len(self.buf) - keep])
                self.buf = self.buf[len(self.buf) - keep:]
                break
            if self.state == "content":
                if self.skip_ws:
                    self.buf = self.buf.lstrip()
                    if not self.buf:
                        break
                    self.skip_ws = False
                tags = [t for t in (self.tool_open if self.decode_call else "", self.think_open if self.may_open_think else "") if t]
                hit = min(((self.buf.find(t), t) for t in tags if t in self.buf), default=None)
                if hit is not None:
                    i, tag = hit
                    before = self.buf[:i]
                    if tag == self.think_open and before.strip():      # a reasoning block only opens the message
                        self.may_open_think = False
                        continue
                    content.append(before.rstrip() if tag == self.tool_open else "")
                    self.buf = self.buf[i + len(tag):]
                    self.state = "tool" if tag == self.tool_open else "thinking"
                    self.may_open_think = False
                    continue
                keep = 0 if done else self._held(self.buf, tags)
                out = self.buf[:len(self.buf) - keep]
                if out.strip():
                    self.may_open_think = False
                content.append(out)
                self.buf = self.buf[len(self.buf) - keep:]
                break
            # state == "tool": wait for the whole body
            end = -1
            if self.tool_close:
                i = self.buf.find(self.tool_close)
                if i >= 0:
                    body, end = self.buf[:i], i + len(self.tool_close)
            elif self.body_end is not None:
                n = self.body_end(self.buf)
                if n >= 0:
                    body, end = self.buf[:n], n
            if end < 0:
                if done:                             # an unterminated call is returned as text, the way it was produced
                    content.append(self.tool_open + self.buf)
                    self.buf = ""
                break
            call = self.decode_call(body) if self.decode_call else None
            if call is not None:
                calls.append(call)
            else:
                content.append(self.tool_open + self.buf[:end])
            self.buf = self.buf[end:]
            self.state, self.skip_ws = "content", True
        return "".join(content), "".join(thinking), calls

    @staticmethod
    def _held(s: str, tags: list[str]) -> int:
        """Characters at the end of ``s`` to keep back: a possible tag prefix and the white space before it."""
        n = max((_overlap(s, t) for t in tags), default=0)
        head = s[:len(s) - n]
        ws = len(head) - len(head.rstrip())
        return n + ws if (n or ws) and tags else 0


# ---------------------------------------------------------------------------------------------------
# tool-call bodies
# ---------------------------------------------------------------------------------------------------
def _json_call(body: str) -> dict[str, Any] | None:
    try:
        obj = json.loads(body.strip())
    except ValueError:
        return None
    if not isinstance(obj, dict) or not isinstance(obj.get("name"), str):
        return None
    args = obj.get("arguments", obj.get("parameters", {}))
    if isinstance(args, str):
        try:
            args = json.loads(args)
        except ValueError:
            return None
    return {"function": {"name": obj["name"], "arguments": args if isinstance(args, dict) else {}}}


def typed_value(raw: str, types: list[str]) -> Any:
    """Text of an XML parameter -> value, by the declared JSON-schema type(s): null first, then the most specific
    type that parses (boolean, integer, number, array, object), string last (model/parsers/qwen3coder.go:292-400)."""
    if raw.lower() == "null":
        return None
    if not types:
        return raw
    ts = set(types)
    only = len(types) == 1
    if "boolean" in ts:
        if raw.lower() in ("true", "false"):
            return raw.lower() == "true"
        if only:
            return False
    if "integer" in ts:
        if re.fullmatch(r"[+-]?\d+", raw):
            return int(raw)
        if only:
            return raw
    if "number" in ts:
        try:
            f = float(raw)
            if f != f or f in (float("inf"), float("-inf")):
                raise ValueError
            return int(f) if f == int(f) else f
        except ValueError:
            if only:
                return raw
    for name, kind in (("array", list), ("object", dict)):
        if name in ts:
            try:
                v = json.loads(raw)
                if isinstance(v, kind):
                    return v
            except ValueError:
                pass
            if only:
                return raw
    return raw


def _schema_types(tools: list[dict[str, Any]] | None, fn: str, param: str) -> list[str]:
    for t in tools or []:
        f = t.get("function", {})
        if f.get("name") == fn:
            p = (f.get("parameters") or {}).get("properties", {}).get(param)
            if isinstance(p, dict):
                ty = p.get("type", [])
                return [ty] if isinstance(ty, str) else [x for x in ty if isinstance(x, str)]
    return []


_FN = re.compile(r"<function=([^>\n]+)>")
_PARAM = re.compile(r"<parameter=([^>\n]+)>(.*?)</parameter>", re.S)


def _xml_call(tools: list[dict[str, Any]] | None) -> Callable[[str], dict[str, Any] | None]:
    def decode(body: str) -> dict[str, Any] | None:
        m = _FN.search(body)
        if m is None:
            return None
        name = m.group(1).strip()
        args: dict[str, Any] = {}
        for pm in _PARAM.finditer(body, m.end()):
            key, val = pm.group(1).strip(), pm.group(2)
            val = val[1:] if val.startswith("\n") else val        # one newline on each side belongs to the format
            val = val[:-1] if val.endswith("\n") else val
            args[key] = typed_value(val, _schema_types(tools, name, key))
        return {"function": {"name": name, "arguments": args}}
    return decode


def _ministral_end(buf: str) -> int:
    """``name[ARGS]{json}``: index just past the balanced JSON object, -1 while it is incomplete."""
    i = buf.find("[ARGS]")
    if i < 0:
        return -1
    j = i + len("[ARGS]")
    while j < len(buf) and buf[j].isspace():
        j += 1
    if j >= len(buf) or buf[j] != "{":
        return -1
    depth, in_str, esc = 0, False, False
    for k in range(j, len(buf)):
        c = buf[k]
        if in_str:
            if esc:
                esc = False
            elif c == "\\":
                esc = True
            elif c == '"':
                in_str = False
        elif c == '"':
            in_str = True
        elif c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                return k + 1
    return -1


def _ministral_call(body: str) -> dict[str, Any] | None:
    name, _, args = body.partition("[ARGS]")
    try:
        obj = json.loads(args)
    except ValueError:
        return None
    return {"function": {"name": name.strip(), "arguments": obj}} if isinstance(obj, dict) and name.strip() else None


# -- functiongemma: call:name{key:value,...} with strings between <escape> marks ----------------------------------
_ESC = "<escape>"


def _fg_split(s: str) -> list[str]:
    """Top-level comma split that respects {...}, [...] and <escape>...<escape> spans."""
    parts, cur, depth, esc, i = [], [], 0, False, 0
    while i < len(s):
        if s.startswith(_ESC, i):
            esc = not esc
            cur.append(_ESC)
            i += len(_ESC)
            continue
        ch = s[i]
        if not esc and ch in "{[":
            depth += 1
        elif not esc and ch in "}]":
            depth -= 1
        if not esc and ch == "," and depth == 0:
            if cur:
                parts.append("".join(cur))
                cur = []
        else:
            cur.append(ch)
        i += 1
    if cur:
        parts.append("".join(cur))
    return parts


def _fg_value(v: str) -> Any:
    if v.startswith(_ESC) and v.endswith(_ESC) and len(v) >= 2 * len(_ESC):
        return v[len(_ESC):-len(_ESC)]
    if v in ("true", "false"):
        return v == "true"
    if re.fullmatch(r"-?\d+", v):
        return int(v)
    if re.fullmatch(r"-?\d+\.\d+(?:[eE][-+]?\d+)?", v):
        return float(v)
    if v.startswith("[") and v.endswith("]"):
        return [_fg_value(x) for x in _fg_split(v[1:-1])]
    if v.startswith("{") and v.endswith("}"):
        return _fg_object(v[1:-1])
    return v


def _fg_object(body: str) -> dict[str, Any]:
    out: dict[str, Any] = {}
    for part in _fg_split(body):
        k, sep, v = part.partition(":")
        if sep:
            out[k] = _fg_value(v)
    return out


_FG_CALL = re.compile(r"call:([^{]+)\{(.*)\}", re.S)


def _functiongemma_call(body: str) -> dict[str, Any] | None:
    m = _FG_CALL.search(body)
    if m is None:
        return None
    return {"function": {"name": m.group(1), "arguments": _fg_object(m.group(2))}}


PARSERS = ("qwen3", "qwen3-thinking", "qwen3-coder", "ministral", "functiongemma", "passthrough")


def parser_for(name: str | None, tools: list[dict[str, Any]] | None = None, think: Any = None,
               prefill: str = "") -> TagStreamParser | None:
    """Parser named by a model's configuration, or None when the name is not a built-in of this module.

    ``think`` is the request's think value (None = unset); ``prefill`` the content of a trailing assistant message
    that the model continues (a reasoning model then continues the answer, not the reasoning block).
    """
    want_tools = bool(tools)
    if name == "passthrough":
        return TagStreamParser()
    if name in ("qwen3", "qwen3-thinking"):
        thinking = name == "qwen3-thinking" and think is not False and not prefill
        return TagStreamParser(think_open="<think>", think_close="</think>", start_thinking=thinking, tool_open="<tool_call>",
                               tool_close="</tool_call>", decode_call=_json_call if want_tools else None)
    if name == "qwen3-coder":
        return TagStreamParser(tool_open="<tool_call>", tool_close="</tool_call>", decode_call=_xml_call(tools))
    if name == "functiongemma":
        return TagStreamParser(tool_open="<start_function_call>", tool_close="<end_function_call>", decode_call=_functiongemma_call)
    if name == "ministral":
        return TagStreamParser(think_open="[THINK]", think_close="[/THINK]", tool_open="[TOOL_CALLS]", tool_close=None,
                               decode_call=_ministral_call, body_end=_ministral_end)
    return None


# ---------------------------------------------------------------------------------------------------
# renderers
# ---------------------------------------------------------------------------------------------------
_QWEN3_CODER_TOOL_HELP = (
    "\n\nIf you choose to call a function ONLY reply in the following format with NO suffix:\n\n<tool_call>\n<function=example_function_name>\n"
    "<parameter=example_parameter_1>\nvalue_1\n</parameter>\n<parameter=example_parameter_2>\nThis is the value for the second parameter\n"
    "that can span\nmultiple lines\n</parameter>\n</function>\n</tool_call>\n\n<IMPORTANT>\nReminder:\n"
    "- Function calls MUST follow the specified format: an inner <function=...></function> block must be nested within "
    "<tool_call></tool_call> XML tags\n- Required parameters MUST be specified\n"
    "- You may provide optional reasoning for your function call in natural language BEFORE the function call, but NOT after\n"
    "- If there is no function call available, answer the question like normal with your current knowledge and do not tell the user "
    "about function calls\n</IMPORTANT>")


def _xml_extra(obj: dict[str, Any], handled: tuple[str, ...]) -> str:
    out = []
    for k, v in obj.items():
        if k in handled or v is None:
            continue
        if isinstance(v, (dict, list)):
            v = json.dumps(v, separators=(",", ":"), ensure_ascii=False)
        elif isinstance(v, bool):
            v = "true" if v else "false"
        out.append(f"\n<{k}>{v}</{k}>")
    return "".join(out)


def _arg_text(v: Any) -> str:
    if v is None:
        return "null"
    if isinstance(v, str):
        return v
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (dict, list)):
        return json.dumps(v, separators=(",", ":"), ensure_ascii=False)
    return str(v)


def render_qwen3_coder(messages: list[dict[str, Any]], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
    """ChatML with XML tool definitions and XML tool calls (model/renderers/qwen3coder.go:63-198): the first system
    message wins, consecutive tool results share one user turn, a trailing assistant message is left open."""
    system = next((m.get("content", "") for m in messages if m.get("role") == "system"), "")
    rest = [m for m in messages if m.get("role") != "system"]
    sb: list[str] = []
    if system or tools:
        sb.append("<|im_start|>system\n")
        sb.append(system or "You are Qwen, a helpful AI assistant that can interact with a computer to solve tasks.")
        if tools:
            sb.append("\n\n# Tools\n\nYou have access to the following functions:\n\n<tools>")
            for t in tools:
                f = t.get("function", {})
                sb.append(f"\n<function>\n<name>{f.get('name', '')}</name>")
                if f.get("description"):
                    sb.append(f"\n<description>{f['description']}</description>")
                sb.append("\n<parameters>")
                params = f.get("parameters") or {}
                for pname, prop in (params.get("properties") or {}).items():
                    sb.append(f"\n<parameter>\n<name>{pname}</name>")
                    ty = prop.get("type")
                    if ty:
                        sb.append(f"\n<type>{ty if isinstance(ty, str) else (ty[0] if len(ty) == 1 else json.dumps(ty, separators=(',', ':')))}</type>")
                    if prop.get("description"):
                        sb.append(f"\n<description>{prop['description']}</description>")
                    sb.append(_xml_extra(prop, ("type", "description")))
                    sb.append("\n</parameter>")
                sb.append(_xml_extra(params, ("type", "properties")))
                sb.append("\n</parameters>\n</function>")
            sb.append("\n</tools>")
            sb.append(_QWEN3_CODER_TOOL_HELP)
        sb.append("<|im_end|>\n")
    for i, m in enumerate(rest):
        last = i == len(rest) - 1
        role, content = m.get("role", "user"), m.get("content", "") or ""
        prefill = last and role == "assistant"
        if role == "assistant":
            sb.append("<|im_start|>assistant\n")
            if m.get("tool_calls"):
                if content:
                    sb.append(content + "\n")
                for c in m["tool_calls"]:
                    f = c.get("function", {})
                    sb.append(f"\n<tool_call>\n<function={f.get('name', '')}>")
                    for k, v in (f.get("arguments") or {}).items():
                        sb.append(f"\n<parameter={k}>\n{_arg_text(v)}\n</parameter>")
                    sb.append("\n</function>\n</tool_call>")
                sb.append("<|im_end|>\n")
                prefill = False
            else:
                sb.append(content)
                if not prefill:
                    sb.append("<|im_end|>\n")
        elif role == "tool":
            if i == 0 or rest[i - 1].get("role") != "tool":
                sb.append("<|im_start|>user")
            sb.append(f"\n<tool_response>\n{content}\n</tool_response>")
            if last or rest[i + 1].get("role") != "tool":
                sb.append("<|im_end|>\n")
        else:
            sb.append(f"<|im_start|>{role}\n{content}<|im_end|>\n")
        if last and not prefill:
            sb.append("<|im_start|>assistant\n")
    return "".join(sb)


def _fg_arg(v: Any) -> str:
    if isinstance(v, str):
        return _ESC + v + _ESC
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, float) and v == int(v):
        return str(int(v))
    if isinstance(v, dict):
        return "{" + ",".join(f"{k}:{_fg_arg(v[k])}" for k in sorted(v)) + "}"
    if isinstance(v, list):
        return "[" + ",".join(_fg_arg(x) for x in v) + "]"
    return str(v)


def render_functiongemma(messages: list[dict[str, Any]], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
    """Gemma turns with function declarations in a developer turn, calls as ``call:name{k:v}`` and tool results as
    ``response:name{...}`` inside the model turn (model/renderers/functiongemma.go:20-125): strings travel between
    ``<escape>`` marks, keys are sorted, types are upper-cased."""
    default = "You can do function calling with the following functions:"
    sb = ["<bos>"]
    system, loop = "", list(messages)
    if loop and loop[0].get("role") in ("system", "developer"):
        system, loop = loop[0].get("content", "") or "", loop[1:]
    if system or tools:
        sb.append("<start_of_turn>developer\n")
        if system:
            sb.append(system.strip())
        if tools:
            if system:
                sb.append("\n")
            if system.strip() != default:
                sb.append(default)
        for t in tools or []:
            f = t.get("function", {})
            sb.append(f"<start_function_declaration>declaration:{f.get('name', '')}{{description:{_ESC}{f.get('description', '')}{_ESC}")
            params = f.get("parameters") or {}
            props, ptype = params.get("properties") or {}, params.get("type") or ""
            if props or ptype or "properties" in params:
                sb.append(",parameters:{")
                items = []
                if props:
                    inner = []
                    for name in sorted(props):
                        pr = props[name] or {}
                        ty = pr.get("type")
                        ty = ty if isinstance(ty, str) else (ty[0] if ty else "")
                        inner.append(f"{name}:{{description:{_ESC}{pr.get('description', '')}{_ESC}" + (f",type:{_ESC}{ty.upper()}{_ESC}" if ty else "") + "}")
                    items.append("properties:{" + ",".join(inner) + "}")
                if params.get("required"):
                    items.append("required:[" + ",".join(_ESC + r + _ESC for r in params["required"]) + "]")
                if ptype:
                    items.append(f"type:{_ESC}{str(ptype).upper()}{_ESC}")
                sb.append(",".join(items) + "}")
            sb.append("}<end_function_declaration>")
        sb.append("<end_of_turn>\n")
    prev = ""
    for i, m in enumerate(loop):
        role, content = m.get("role", "user"), m.get("content", "") or ""
        if role == "assistant":
            if prev != "tool_response":
                sb.append("<start_of_turn>model\n")
            prev = ""
            if content:
                sb.append(content.strip())
            calls = m.get("tool_calls") or []
            for c in calls:
                f = c.get("function", {})
                args = f.get("arguments") or {}
                sb.append("<start_function_call>call:" + f.get("name", "") + "{" + ",".join(f"{k}:{_fg_arg(args[k])}" for k in sorted(args)) + "}<end_function_call>")
            if calls and i + 1 < len(loop) and loop[i + 1].get("role") == "tool":
                sb.append("<start_function_response>")
                prev = "tool_call"
            else:
                sb.append("<end_of_turn>\n")
        elif role == "tool":
            name = ""
            for j in range(i - 1, -1, -1):          # the call this result answers: n-th result after the last assistant turn with calls
                if loop[j].get("role") == "assistant" and loop[j].get("tool_calls"):
                    n = sum(1 for k in range(j + 1, i) if loop[k].get("role") == "tool")
                    if n < len(loop[j]["tool_calls"]):
                        name = loop[j]["tool_calls"][n].get("function", {}).get("name", "")
                    break
            if prev != "tool_call":
                sb.append("<start_function_response>")
            sb.append("response:" + name + "{" + _fg_arg(content) + "}<end_function_response>")
            prev = "tool_response"
        else:
            if role != "user" or prev != "tool_response":
                sb.append(f"<start_of_turn>{role}\n")
            prev = ""
            sb.append(content.strip() + "<end_of_turn>\n")
    if prev != "tool_response":
        sb.append("<start_of_turn>model\n")
    return "".join(sb)


RENDERERS: dict[str, Callable[..., str]] = {"qwen3-coder": render_qwen3_coder, "functiongemma": render_functiongemma}


def renderer_for(name: str | None) -> Callable[..., str] | None:
    return RENDERERS.get(name or "")
