"""Prompt renderers for model families whose chat format is code, not a template (Modelfile ``RENDERER``).

The reference has one hand-written Go loop per family (model/renderers/renderer.go:56-125).  Here a conversation is
first put into a normal form that every family shares (:class:`Conversation`: where the system text comes from, runs
of tool results folded into one turn with the name of the call each result answers, the turn the last real question
is in, whether the model continues a trailing assistant message) and a family is a :class:`Dialect`: a handful of
small methods that print one piece each (the head with system text and tool declarations, a user turn, an assistant
turn, a run of tool results, the cue that makes the model speak).  ``Dialect.render`` strings the pieces together, so
the order of a prompt is written down once.

===================  ==============================================================================================
name                 format
===================  ==============================================================================================
qwen3-coder          ChatML, tools declared as XML, calls as ``<function=..><parameter=..>`` (qwen3coder.go:63-198)
qwen3-vl-instruct    ChatML, tools declared as JSON lines, calls as JSON in ``<tool_call>`` (qwen3vl.go:40-148)
qwen3-vl-thinking    the same with ``<think>`` blocks kept after the last question
qwen3.5 / ornith     ChatML, JSON declarations with XML calls, trimmed content (qwen35.go:210-360)
qwen3.8              the same with merged instructions and a reasoning-effort sentence (qwen35.go:117-208)
cogito               DeepSeek marks, tools as fenced JSON in the system text (cogito.go:18-132)
deepseek3.1          DeepSeek marks, ``</think>`` closes an absent reasoning block (deepseek3.go:26-160)
olmo3 / olmo3.1      ChatML, ``<functions>`` in the system turn, Python-style calls (olmo3.go:27-158)
olmo3-think (+32b)   ChatML, no tools, cue ends in ``<think>`` (olmo3_think.go:32-87)
glm-4.6 / glm-4.7    ``<|user|>`` marks, calls as ``<arg_key>/<arg_value>`` pairs (glm46.go:17-113, glm47.go:43-108)
lfm2 / lfm2-thinking ChatML behind ``<|startoftext|>``, tool list in the system turn, Python-style call list (lfm2.go:222-335)
cohere               Command turn marks, tool section and action / result lists as JSON (cohere.go:77-226)
functiongemma        Gemma turns, declarations and calls in the ``call:name{k:v}`` notation (functiongemma.go:20-125)
===================  ==============================================================================================
"""
from __future__ import annotations

import datetime
import json
import re
from dataclasses import dataclass, field
from typing import Any, Callable

Message = dict[str, Any]


# ---------------------------------------------------------------------------------------------------
# JSON the way the reference's encoder prints it
# ---------------------------------------------------------------------------------------------------
def _plain(v: Any, sort: bool | None) -> Any:
    """Integral floats print as integers.  ``sort``: True prints every map with sorted keys (a value of unknown shape),
    None keeps the order of the outermost map only (call arguments: the order they were given in), False keeps all."""
    if isinstance(v, float) and v == int(v) and abs(v) < 1e15:
        return int(v)
    if isinstance(v, dict):
        below = True if sort is None else sort
        return {k: _plain(v[k], below) for k in (sorted(v) if sort else v)}
    if isinstance(v, (list, tuple)):
        return [_plain(x, True if sort is None else sort) for x in v]
    return v


def go_json(v: Any, *, spaced: bool = False, indent: int | None = None, sort: bool | None = False, html: bool = True) -> str:
    """Compact JSON with ``<``, ``>``, ``&`` and the two Unicode line separators escaped, as Go's ``json.Marshal`` does;
    ``spaced`` puts one blank after every ``:`` and ``,`` outside strings, ``indent`` gives the multi-line form."""
    seps = None if indent is not None else ((", ", ": ") if spaced else (",", ":"))
    s = json.dumps(_plain(v, sort), ensure_ascii=False, separators=seps, indent=indent)
    if not html:                                # an encoder with HTML escaping switched off
        return s
    for ch, esc in (("<", "\\u003c"), (">", "\\u003e"), ("&", "\\u0026"), ("\u2028", "\\u2028"), ("\u2029", "\\u2029")):
        s = s.replace(ch, esc)
    return s


def args_json(args: dict[str, Any], spaced: bool = False) -> str:
    """Call arguments: the outer keys in the order of the call, maps inside them with sorted keys."""
    return go_json(args, spaced=spaced, sort=None)


def _types(prop: dict[str, Any]) -> list[str]:
    ty = prop.get("type")
    return [ty] if isinstance(ty, str) else [t for t in (ty or []) if isinstance(t, str)]


def _property(p: Any) -> Any:
    """One parameter's schema in the field order of the wire type (api/types.go:418-426); a one-element type list
    prints as a plain string."""
    if not isinstance(p, dict):
        return p
    out: dict[str, Any] = {}
    if p.get("anyOf"):
        out["anyOf"] = [_property(x) for x in p["anyOf"]]
    ty = _types(p)
    if ty:
        out["type"] = ty[0] if len(ty) == 1 else ty
    if p.get("items") is not None:
        out["items"] = _plain(p["items"], True)
    if p.get("description"):
        out["description"] = p["description"]
    if p.get("enum"):
        out["enum"] = _plain(p["enum"], True)
    if isinstance(p.get("properties"), dict):
        out["properties"] = {k: _property(v) for k, v in p["properties"].items()}
    if p.get("required"):
        out["required"] = list(p["required"])
    return out


def parameters_schema(params: dict[str, Any] | None) -> dict[str, Any]:
    """A function's parameter block in wire order: type, $defs, items, required, properties (api/types.go:473-479)."""
    params = params or {}
    out: dict[str, Any] = {"type": params.get("type", "")}
    for key in ("$defs", "items"):
        if params.get(key) is not None:
            out[key] = _plain(params[key], True)
    if params.get("required"):
        out["required"] = list(params["required"])
    props = params.get("properties")
    out["properties"] = {k: _property(v) for k, v in props.items()} if isinstance(props, dict) else None
    return out


def tool_schema(tool: dict[str, Any]) -> dict[str, Any]:
    """A tool declaration in wire order (api/types.go:305-309, :486-490), whatever order the client sent."""
    f = tool.get("function") or {}
    out: dict[str, Any] = {"type": tool.get("type", "function")}
    if tool.get("items") is not None:
        out["items"] = _plain(tool["items"], True)
    fn: dict[str, Any] = {"name": f.get("name", "")}
    if f.get("description"):
        fn["description"] = f["description"]
    fn["parameters"] = parameters_schema(f.get("parameters"))
    out["function"] = fn
    return out


def think_on(think: Any, default: bool) -> bool:
    """The request's think value as a switch: unset -> ``default``, a level name ("low", "high", ...) counts as on."""
    if think is None:
        return default
    return bool(think)


# ---------------------------------------------------------------------------------------------------
# normal form of a conversation
# ---------------------------------------------------------------------------------------------------
@dataclass
class Turn:
    role: str                                   # "user", "assistant", "tool" (a run of results) or any other role kept in place
    content: str = ""
    thinking: str = ""
    calls: list[tuple[str, dict[str, Any]]] = field(default_factory=list)     # assistant: (function name, arguments)
    results: list[tuple[str, str]] = field(default_factory=list)              # tool: (name of the answered call, content)
    call_ids: list[str] = field(default_factory=list)                         # assistant: the id each call travelled with ("" if none)
    result_ids: list[str] = field(default_factory=list)                       # tool: the call id each result names
    images: int = 0
    pos: int = 0                                # index among the turns
    first_image: int = 0                        # number of images in the turns before this one


class Conversation:
    """``system``: "leading" takes the text of messages[0] if that is a system message (``lead_roles``) and leaves later
    ones in place as turns; "first" takes the first system message wherever it is and drops the others; "join" takes
    all of them, joined by blank lines; "inline" leaves every message where it is.  ``system_text`` is None when the
    conversation has none."""

    def __init__(self, messages: list[Message], system: str = "leading", lead_roles: tuple[str, ...] = ("system",),
                 drop: tuple[str, ...] = ()):
        self.system_text: str | None = None
        msgs = [m for m in messages if m.get("role") not in drop]
        if system == "leading":
            if msgs and msgs[0].get("role") in lead_roles:
                self.system_text, msgs = msgs[0].get("content") or "", msgs[1:]
        elif system in ("first", "join"):
            texts = [m.get("content") or "" for m in msgs if m.get("role") in lead_roles]
            if texts:
                self.system_text = texts[0] if system == "first" else "\n\n".join(texts)
            msgs = [m for m in msgs if m.get("role") not in lead_roles]
        self.turns: list[Turn] = []
        images = 0
        pending: list[str] = []                 # names of the calls of the last assistant turn that no result has answered yet
        for m in msgs:
            role = m.get("role") or "user"
            if role == "tool":
                name = (pending.pop(0) if pending else "") or m.get("tool_name") or m.get("name") or ""
                if not self.turns or self.turns[-1].role != "tool":
                    self.turns.append(Turn("tool", pos=len(self.turns), first_image=images))
                self.turns[-1].results.append((name, m.get("content") or ""))
                self.turns[-1].result_ids.append(m.get("tool_call_id") or "")
                continue
            t = Turn(role, m.get("content") or "", m.get("thinking") or "", pos=len(self.turns), first_image=images,
                     images=len(m.get("images") or []))
            for c in m.get("tool_calls") or []:
                f = c.get("function") or {}
                t.calls.append((f.get("name", ""), f.get("arguments") or {}))
                t.call_ids.append(c.get("id") or "")
            if role == "assistant" and t.calls:
                pending = [n for n, _ in t.calls]
            images += t.images
            self.turns.append(t)

    @property
    def last(self) -> Turn | None:
        return self.turns[-1] if self.turns else None

    @property
    def continued(self) -> Turn | None:
        """The trailing assistant message the model is to continue (one without calls), if the conversation ends in one."""
        t = self.last
        return t if t is not None and t.role == "assistant" and not t.calls else None

    def last_user(self, default: int = -1, real: Callable[[Turn], bool] | None = None) -> int:
        for t in reversed(self.turns):
            if t.role == "user" and (real is None or real(t)):
                return t.pos
        return default

    def before(self, t: Turn) -> Turn | None:
        return self.turns[t.pos - 1] if t.pos > 0 else None

    def after(self, t: Turn) -> Turn | None:
        return self.turns[t.pos + 1] if t.pos + 1 < len(self.turns) else None


@dataclass
class Ctx:
    conv: Conversation
    tools: list[dict[str, Any]]
    think: Any
    memo: dict[str, Any] = field(default_factory=dict)


class Dialect:
    """One chat format.  Subclasses print pieces; ``render`` orders them: head, the turns, cue."""

    system = "leading"
    lead_roles: tuple[str, ...] = ("system",)
    drop: tuple[str, ...] = ()
    bos = ""                                    # the text the prompt begins with, for callers that must not add a second one

    def render(self, messages: list[Message], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
        x = Ctx(Conversation(messages, self.system, self.lead_roles, self.drop), list(tools or []), think)
        self.prepare(x)
        out = [self.head(x)]
        for t in x.conv.turns:
            out.append(getattr(self, "turn_" + t.role, self.turn_other)(t, x))
        out.append(self.cue(x))
        return "".join(out)

    __call__ = render

    def prepare(self, x: Ctx) -> None:
        pass

    def head(self, x: Ctx) -> str:
        return ""

    def turn_other(self, t: Turn, x: Ctx) -> str:
        return ""

    def cue(self, x: Ctx) -> str:
        return ""


# ---------------------------------------------------------------------------------------------------
# ChatML family
# ---------------------------------------------------------------------------------------------------
class ChatML(Dialect):
    """``<|im_start|>role\\n ... <|im_end|>\\n`` turns; a run of tool results travels as one user turn of
    ``<tool_response>`` blocks; a trailing assistant message stays open."""

    opener, closer = "<|im_start|>", "<|im_end|>\n"

    def block(self, role: str, body: str, close: bool = True) -> str:
        return f"{self.opener}{role}\n{body}" + (self.closer if close else "")

    def turn_other(self, t: Turn, x: Ctx) -> str:
        return self.block(t.role, t.content)

    turn_user = turn_other

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return f"{self.opener}user" + "".join(f"\n<tool_response>\n{c}\n</tool_response>" for _, c in t.results) + self.closer

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        return self.block("assistant", t.content + self.calls(t), close=t is not x.conv.continued)

    def calls(self, t: Turn) -> str:
        return ""

    def cue(self, x: Ctx) -> str:
        return "" if x.conv.continued is not None or not x.conv.turns else f"{self.opener}assistant\n"


_QWEN3_CODER_CALL_FORMAT = (
    "\n\nIf you choose to call a function ONLY reply in the following format with NO suffix:\n\n<tool_call>\n<function=example_function_name>\n"
    "<parameter=example_parameter_1>\nvalue_1\n</parameter>\n<parameter=example_parameter_2>\nThis is the value for the second parameter\n"
    "that can span\nmultiple lines\n</parameter>\n</function>\n</tool_call>\n\n<IMPORTANT>\nReminder:\n"
    "- Function calls MUST follow the specified format: an inner <function=...></function> block must be nested within "
    "<tool_call></tool_call> XML tags\n- Required parameters MUST be specified\n"
    "- You may provide optional reasoning for your function call in natural language BEFORE the function call, but NOT after\n"
    "- If there is no function call available, answer the question like normal with your current knowledge and do not tell the user "
    "about function calls\n</IMPORTANT>")


def _xml_scalar(v: Any) -> str:
    if v is None:
        return "null"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (dict, list)):
        return json.dumps(v, separators=(",", ":"), ensure_ascii=False)
    return str(v)


def _xml_fields(obj: dict[str, Any], skip: tuple[str, ...]) -> str:
    """Schema keys beyond the ones with a tag of their own, one ``<key>value</key>`` line each."""
    return "".join(f"\n<{k}>{_xml_scalar(v)}</{k}>" for k, v in obj.items() if k not in skip and v is not None)


class Qwen3Coder(ChatML):
    system = "first"
    default_system = "You are Qwen, a helpful AI assistant that can interact with a computer to solve tasks."

    def head(self, x: Ctx) -> str:
        if not (x.conv.system_text or x.tools):
            return ""
        body = x.conv.system_text or self.default_system
        if x.tools:
            body += "\n\n# Tools\n\nYou have access to the following functions:\n\n<tools>" + "".join(map(self.declare, x.tools)) + "\n</tools>"
            body += _QWEN3_CODER_CALL_FORMAT
        return self.block("system", body)

    @staticmethod
    def declare(tool: dict[str, Any]) -> str:
        f = tool.get("function") or {}
        params = f.get("parameters") or {}
        out = f"\n<function>\n<name>{f.get('name', '')}</name>"
        if f.get("description"):
            out += f"\n<description>{f['description']}</description>"
        out += "\n<parameters>"
        for name, prop in (params.get("properties") or {}).items():
            ty = prop.get("type")
            out += f"\n<parameter>\n<name>{name}</name>"
            if ty:
                out += "\n<type>" + (ty if isinstance(ty, str) else ty[0] if len(ty) == 1 else json.dumps(ty, separators=(",", ":"))) + "</type>"
            if prop.get("description"):
                out += f"\n<description>{prop['description']}</description>"
            out += _xml_fields(prop, ("type", "description")) + "\n</parameter>"
        return out + _xml_fields(params, ("type", "properties")) + "\n</parameters>\n</function>"

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        if not t.calls:
            return super().turn_assistant(t, x)
        return self.block("assistant", (t.content + "\n" if t.content else "") + self.calls(t))

    def calls(self, t: Turn) -> str:
        return "".join(f"\n<tool_call>\n<function={name}>" + "".join(f"\n<parameter={k}>\n{_xml_scalar(v)}\n</parameter>" for k, v in args.items())
                       + "\n</function>\n</tool_call>" for name, args in t.calls)


_QWEN_JSON_TOOLS_INTRO = ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                          "You are provided with function signatures within <tools></tools> XML tags:\n<tools>")
_QWEN_JSON_TOOLS_OUTRO = ("\n</tools>\n\nFor each function call, return a json object with function name and arguments within <tool_call></tool_call> XML tags:\n"
                          "<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n</tool_call>")


def image_tagged(content: str, n: int, first: int) -> str:
    """``[img-N]`` marks for a message's ``n`` images, numbered from ``first``: explicit ``[img]`` marks are numbered in
    order, images without one go in front (model/renderers/image_tags.go:13-39); text that already carries numbered marks
    is left alone."""
    if n == 0 or "[img-" in content:
        return content
    front = ""
    for i in range(first, first + n):
        if "[img]" in content:
            content = content.replace("[img]", f"[img-{i}]", 1)
        else:
            front += f"[img-{i}]"
    return front + (" " if front and content and not content[0].isspace() else "") + content


class Qwen3VL(ChatML):
    """Text path of the vision-language checkpoints.  Reasoning of earlier rounds is dropped: only assistant turns after
    the last real question (a user turn that is not a wrapped tool result) keep their ``<think>`` block."""

    def __init__(self, thinking: bool, image_tags: bool = True, empty_block_when_off: bool = False):
        self.thinking, self.image_tags, self.empty_block_when_off = thinking, image_tags, empty_block_when_off

    def text(self, t: Turn) -> str:
        if self.image_tags:
            return image_tagged(t.content, t.images, t.first_image)
        return "<|vision_start|><|image_pad|><|vision_end|>" * t.images + t.content

    def prepare(self, x: Ctx) -> None:
        def real(t: Turn) -> bool:
            c = self.text(t)
            return not (c.startswith("<tool_response>") and c.endswith("</tool_response>"))
        x.memo["question"] = x.conv.last_user(default=len(x.conv.turns) - 1, real=real)
        x.memo["thinking"] = think_on(x.think, self.thinking)

    def head(self, x: Ctx) -> str:
        sys = x.conv.system_text
        if x.tools:
            body = (sys + "\n\n" if sys is not None else "") + _QWEN_JSON_TOOLS_INTRO
            body += "".join("\n" + go_json(tool_schema(t), spaced=True) for t in x.tools) + _QWEN_JSON_TOOLS_OUTRO
            return self.block("system", body)
        return self.block("system", sys) if sys is not None else ""

    def turn_other(self, t: Turn, x: Ctx) -> str:
        return self.block(t.role, self.text(t)) if t.role in ("user", "system") else ""

    turn_user = turn_other

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return super().turn_tool(t, x)

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        content = self.text(t)
        body = content
        if x.memo["thinking"] and t.pos > x.memo["question"] and (t is x.conv.last or t.thinking):
            body = "<think>\n" + t.thinking.strip("\n") + ("\n</think>\n\n" + content.lstrip("\n") if content else "")
        for j, (name, args) in enumerate(t.calls):
            body += ("\n" if j or content else "") + '<tool_call>\n{"name": "' + name + '", "arguments": ' + args_json(args, spaced=True) + "}\n</tool_call>"
        return self.block("assistant", body, close=t is not x.conv.last)

    def cue(self, x: Ctx) -> str:
        last = x.conv.last
        if last is None or last.role == "assistant":
            return ""
        return f"{self.opener}assistant\n" + ("<think>\n" if x.memo["thinking"] else "<think>\n\n</think>\n\n" if self.empty_block_when_off else "")


class RenderError(ValueError):
    """The conversation cannot be rendered for this family (the request is at fault)."""


_QWEN35_TOOLS_OUTRO = "\n</tools>" + _QWEN3_CODER_CALL_FORMAT
_QWEN38_EFFORT = {
    "high": ("Reasoning effort is set to xhigh. Please think carefully through the task, validate key assumptions, consider plausible alternatives, "
             "and prioritize correctness, consistency, and clarity in the final answer."),
    "low": "Reasoning effort is set to low. Keep your thinking brief and focused, moving directly to the conclusion without unnecessary elaboration.",
    "medium": "",
}
_QWEN38_EFFORT["max"] = _QWEN38_EFFORT["high"]


class Qwen35(Qwen3VL):
    """ChatML with JSON tool declarations but XML calls; content is trimmed; the system text follows the tool section.

    ``always_block``: every stored assistant turn is printed with a ``<think>`` block (empty if it has no reasoning), not only
    the turns after the last question.  ``effort`` (the 3.8 spelling): system and developer messages are merged into one
    leading system turn, a sentence about the reasoning effort opens it, reasoning is never dug out of stored content, and
    a conversation without a real question is refused."""

    def __init__(self, always_block: bool = False, effort: bool = False, image_tags: bool = True):
        super().__init__(thinking=True, image_tags=image_tags, empty_block_when_off=True)
        self.always_block, self.effort = always_block, effort

    def render(self, messages, tools=None, think=None):
        if self.effort:
            messages = self._merged_instructions(messages)
            if not messages:
                raise RenderError("no messages provided")
        return super().render(messages, tools, think)

    @staticmethod
    def _merged_instructions(messages: list[Message]) -> list[Message]:
        lead = [m for m in messages if m.get("role") in ("system", "developer")]
        if any(m.get("images") for m in lead):
            raise RenderError("system message cannot contain images")
        if not lead or (len(lead) == 1 and messages[0].get("role") == "system"):
            return messages
        text = "\n\n".join(t for t in ((m.get("content") or "").strip() for m in lead) if t)
        return [{"role": "system", "content": text}] + [m for m in messages if m.get("role") not in ("system", "developer")]

    def text(self, t: Turn) -> str:
        return super().text(t).strip()

    def prepare(self, x: Ctx) -> None:
        super().prepare(x)
        x.memo["thinking"] = self.thinking if x.think is None else think_on(x.think, True) and x.think is not False
        x.memo["effort"] = ""
        if self.effort:
            if x.think is not None and not isinstance(x.think, bool) and x.think not in _QWEN38_EFFORT:
                raise RenderError(f"unsupported reasoning effort {x.think!r}")
            x.memo["effort"] = _QWEN38_EFFORT["high"] if x.think is None else "" if isinstance(x.think, bool) else _QWEN38_EFFORT[x.think]
            if not any(t.role == "user" and not self._wrapped(self.text(t)) for t in x.conv.turns):
                raise RenderError("no user query found in messages")

    @staticmethod
    def _wrapped(c: str) -> bool:
        return c.startswith("<tool_response>") and c.endswith("</tool_response>")

    def head(self, x: Ctx) -> str:
        sys = None if x.conv.system_text is None else x.conv.system_text.strip()
        effort = x.memo["effort"]
        if x.tools:
            body = (effort + "\n\n" if effort else "") + "# Tools\n\nYou have access to the following functions:\n\n<tools>"
            body += "".join("\n" + go_json(tool_schema(t), spaced=True) for t in x.tools) + _QWEN35_TOOLS_OUTRO
            return self.block("system", body + ("\n\n" + sys if sys else ""))
        if sys is not None:
            if self.effort and not sys and not effort:
                return ""
            return self.block("system", effort + ("\n\n" if effort and sys else "") + sys)
        return self.block("system", effort) if effort else ""

    def turn_other(self, t: Turn, x: Ctx) -> str:
        if t.role in ("user", "system") or self.effort:
            return self.block(t.role, self.text(t))
        return ""

    turn_user = turn_other

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return f"{self.opener}user" + "".join(f"\n<tool_response>\n{c.strip()}\n</tool_response>" for _, c in t.results) + self.closer

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        content = self.text(t)
        block = self.always_block or (x.memo["thinking"] and t.pos > x.memo["question"])
        reasoning = ""
        if block and t.thinking:
            reasoning = t.thinking.strip()
        elif not self.effort and "</think>" in content:          # reasoning that an older client left inside the content
            before, _, after = content.partition("</think>")
            reasoning, content = before.rpartition("<think>")[2].strip(), after.lstrip("\n")
        body = f"<think>\n{reasoning}\n</think>\n\n{content}" if block else content
        for j, (name, args) in enumerate(t.calls):
            body += ("\n\n" if content.strip() else "") if j == 0 else "\n"
            body += f"<tool_call>\n<function={name}>\n" + "".join(f"<parameter={k}>\n{_xml_scalar(v)}\n</parameter>\n" for k, v in args.items())
            body += "</function>\n</tool_call>"
        return self.block("assistant", body, close=t is not x.conv.last)


class LFM2(ChatML):
    """ChatML behind ``<|startoftext|>``; tools as a JSON list in the system turn, calls as ``[name(k=json, ...)]`` between call
    marks in front of the content, every tool result in a turn of its own between response marks.  Reasoning of stored turns
    is cut away except in the last assistant turn, unless a thinking variant was asked to think."""

    bos = "<|startoftext|>"

    def __init__(self, thinking: bool, image_tags: bool = True):
        self.thinking, self.image_tags = thinking, image_tags

    def prepare(self, x: Ctx) -> None:
        x.memo["keep"] = self.thinking and x.think is not None and think_on(x.think, False)
        x.memo["last_assistant"] = max((t.pos for t in x.conv.turns if t.role == "assistant"), default=-1)

    def text(self, t: Turn) -> str:
        if not t.images:
            return t.content
        if self.image_tags:
            return image_tagged(t.content, t.images, t.first_image)
        return t.content if "<image>" in t.content else "<image>" * t.images + t.content

    def head(self, x: Ctx) -> str:
        sys = x.conv.system_text or ""
        if x.tools:
            listing = ", ".join(go_json(self.schema(t), spaced=True, html=False) for t in x.tools)
            sys += ("\n" if sys else "") + "List of tools: <|tool_list_start|>[" + listing + "]<|tool_list_end|>"
        return self.bos + (self.block("system", sys) if sys else "")

    @staticmethod
    def schema(tool: dict[str, Any]) -> dict[str, Any]:
        full = tool_schema(tool)
        return full["function"] if full["function"]["name"] else full

    def turn_other(self, t: Turn, x: Ctx) -> str:
        return self.block(t.role, self.text(t))

    turn_user = turn_other

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return "".join(self.block("tool", c if "<|tool_response_start|>" in c else f"<|tool_response_start|>{c}<|tool_response_end|>") for _, c in t.results)

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        content = self.text(t)
        if t.calls and "<|tool_call_start|>" not in content:
            calls = ",".join(name + "(" + ",".join(f"{k}={go_json(args[k], spaced=True, html=False, sort=True)}" for k in sorted(args)) + ")" for name, args in t.calls)
            content = "<|tool_call_start|>[" + calls + "]<|tool_call_end|>" + ("\n" + content if content.strip() else content)
        if self.thinking and t.thinking and "</think>" not in content:
            content = f"<think>{t.thinking}</think>{content}"
        if not x.memo["keep"] and t.pos != x.memo["last_assistant"] and "</think>" in content:
            content = content.rpartition("</think>")[2].strip()
        return self.block("assistant", content, close=t is not x.conv.last)

    def cue(self, x: Ctx) -> str:
        last = x.conv.last
        return "" if last is not None and last.role == "assistant" else f"{self.opener}assistant\n"


_OLMO3_WITH_FUNCTIONS = ("You are provided with function signatures within <functions></functions> XML tags. You may call one or more functions to assist "
                         "with the user query. Output any function calls within <function_calls></function_calls> XML tags. Do not make assumptions about "
                         "what values to plug into functions.")
_OLMO31_IDENTITY = ("You are Olmo, a helpful AI assistant built by Ai2. Your date cutoff is December 2024, and your model weights are available at "
                    "https://huggingface.co/allenai.")


class Olmo3(ChatML):
    system = "first"

    def __init__(self, extended: bool):
        self.default_system = _OLMO31_IDENTITY + " " if extended else "You are a helpful function-calling AI assistant. "

    def head(self, x: Ctx) -> str:
        functions = "<functions>" + go_json([tool_schema(t) for t in x.tools], spaced=True) + "</functions>" if x.tools else ""
        if x.conv.system_text is not None:
            return self.block("system", x.conv.system_text + functions)
        if x.tools:
            return self.block("system", self.default_system + _OLMO3_WITH_FUNCTIONS + functions)
        return self.block("system", self.default_system + "You do not currently have access to any functions. <functions></functions>")

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return "".join(self.block("environment", c) for _, c in t.results)

    def turn_other(self, t: Turn, x: Ctx) -> str:
        return self.block("user", t.content) if t.role == "user" else ""

    turn_user = turn_other

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        return self.block("assistant", t.content + self.calls(t), close=bool(t.calls) or t is not x.conv.last)

    def calls(self, t: Turn) -> str:
        """``name(key="value", n=1)``, keys sorted, one call per line."""
        if not t.calls:
            return ""
        lines = [name + "(" + ", ".join(f"{k}={go_json(args[k], sort=True)}" for k in sorted(args)) + ")" for name, args in t.calls]
        return "<function_calls>" + "\n".join(lines) + "</function_calls>"

    def cue(self, x: Ctx) -> str:
        t = x.conv.continued
        return "" if t is not None and t.content else f"{self.opener}assistant\n"


class Olmo3Think(ChatML):
    system, drop = "first", ("tool",)

    def __init__(self, default_system: str):
        self.default_system = default_system

    def head(self, x: Ctx) -> str:
        if x.conv.system_text is None:
            return self.block("system", self.default_system)
        return self.block("system", x.conv.system_text + " You do not currently have access to any functions. <functions></functions>")

    def turn_other(self, t: Turn, x: Ctx) -> str:
        return self.block(t.role, t.content) if t.role in ("user", "assistant") else ""

    turn_user = turn_assistant = turn_other

    def cue(self, x: Ctx) -> str:
        return f"{self.opener}assistant\n<think>"


# ---------------------------------------------------------------------------------------------------
# DeepSeek marks
# ---------------------------------------------------------------------------------------------------
class DeepSeekMarks(Dialect):
    bos = "<｜begin▁of▁sentence｜>"
    eos = "<｜end▁of▁sentence｜>"
    user, assistant = "<｜User｜>", "<｜Assistant｜>"

    @staticmethod
    def call_block(calls: list[str]) -> str:
        return "<｜tool▁calls▁begin｜>" + "".join(calls) + "<｜tool▁calls▁end｜>"


class Cogito(DeepSeekMarks):
    """Reasoning is switched on by a sentence in front of the system text and only when the request asks for it."""

    identity = "You are Cogito, an AI assistant created by Deep Cogito, which is an AI research lab based in San Francisco."

    def prepare(self, x: Ctx) -> None:
        x.memo["thinking"] = think_on(x.think, False)

    def head(self, x: Ctx) -> str:
        sys, deep = x.conv.system_text, x.memo["thinking"]
        text = ("Enable deep thinking subroutine.\n\n" if deep else "") + self.identity
        if sys:
            text += "\n\n" + sys + ("\n\n" if deep else "")
        if x.tools:
            text += "\nYou have the following functions available:\n"
            text += "".join("```json\n" + go_json(tool_schema(t), indent=4) + "\n```\n" for t in x.tools)
        return self.bos + text

    def turn_user(self, t: Turn, x: Ctx) -> str:
        return self.user + t.content + self.assistant

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        if not t.calls:
            return t.content + self.eos
        calls = ["<｜tool▁call▁begin｜>function<｜tool▁sep｜>" + name + "\n```json\n" + args_json(args) + "\n```<｜tool▁call▁end｜>" for name, args in t.calls]
        return t.content + "<｜tool▁calls▁begin｜>" + "\n".join(calls) + "<｜tool▁calls▁end｜>" + self.eos

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return "<｜tool▁outputs▁begin｜>" + "\n".join(f"<｜tool▁output▁begin｜>{c}<｜tool▁output▁end｜>" for _, c in t.results) + "<｜tool▁outputs▁end｜>"

    def cue(self, x: Ctx) -> str:
        speakers = [t for t in x.conv.turns if t.role in ("user", "assistant", "tool")]
        out = "" if speakers and speakers[-1].role == "user" else self.assistant
        return out + ("<think>\n" if x.memo["thinking"] else "")


_DEEPSEEK_TOOL_FORMAT = (
    "\nIMPORTANT: ALWAYS adhere to this exact format for tool use:\n"
    "<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>tool_call_name<｜tool▁sep｜>tool_call_arguments<｜tool▁call▁end｜>{{additional_tool_calls}}<｜tool▁calls▁end｜>\n\n"
    "Where:\n\n- `tool_call_name` must be an exact match to one of the available tools\n"
    "- `tool_call_arguments` must be valid JSON that strictly follows the tool's Parameters Schema\n"
    "- For multiple tool calls, chain them directly without separators or spaces\n")


class DeepSeek31(DeepSeekMarks):
    """The assistant mark is printed by the turn that follows a user turn, together with ``<think>`` (a reasoning block
    follows) or ``</think>`` (none does); stored answers lose everything up to their own ``</think>``."""

    system = "join"

    def prepare(self, x: Ctx) -> None:
        x.memo["thinking"] = think_on(x.think, False)
        x.memo["question"] = x.conv.last_user()

    def head(self, x: Ctx) -> str:
        out = self.bos + (x.conv.system_text or "")
        if x.tools:
            out += "\n\n## Tools\nYou have access to the following tools:\n"
            for t in x.tools:
                f = t.get("function") or {}
                out += f"\n### {f.get('name', '')}\nDescription: {f.get('description', '')}\n\nParameters: {go_json(parameters_schema(f.get('parameters')))}\n"
            out += _DEEPSEEK_TOOL_FORMAT
        return out

    def turn_user(self, t: Turn, x: Ctx) -> str:
        return self.user + t.content

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        prev = x.conv.before(t)
        asked = prev is not None and prev.role == "user"
        if t.calls:
            calls = [f"<｜tool▁call▁begin｜>{name}<｜tool▁sep｜>{args_json(args)}<｜tool▁call▁end｜>" for name, args in t.calls]
            return (self.assistant + "</think>" if asked else "") + t.content + self.call_block(calls) + self.eos
        out = ""
        if asked:
            out = self.assistant + ("<think>" if t.thinking and x.memo["thinking"] and t.pos > x.memo["question"] else "</think>")
        content = t.content
        if not (prev is not None and prev.role == "tool"):
            content = content.split("</think>", 1)[-1]
        return out + content + self.eos

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return "".join(f"<｜tool▁output▁begin｜>{c}<｜tool▁output▁end｜>" for _, c in t.results)

    def cue(self, x: Ctx) -> str:
        last = x.conv.last
        if last is None or last.role != "user":
            return ""
        return self.assistant + ("<think>" if x.memo["thinking"] else "</think>")


# ---------------------------------------------------------------------------------------------------
# Cohere
# ---------------------------------------------------------------------------------------------------
class Cohere(Dialect):
    """Command models: turns between ``<|START_OF_TURN_TOKEN|><|ROLE_TOKEN|>`` and ``<|END_OF_TURN_TOKEN|>``, text between text
    marks, a tool section in the system turn even when it is empty, calls as a JSON action list whose ids are the running
    number of the call in the conversation, results as a JSON list in a system turn."""

    bos = "<BOS_TOKEN>"
    T0, T1 = "<|START_OF_TURN_TOKEN|>", "<|END_OF_TURN_TOKEN|>"

    def render(self, messages, tools=None, think=None):
        alias = {"chatbot": "assistant"}
        messages = [{**m, "role": alias.get(str(m.get("role", "")).lower(), str(m.get("role", "")).lower())} for m in messages]
        return super().render(messages, tools, think)

    def prepare(self, x: Ctx) -> None:
        x.memo["numbers"], x.memo["next"] = {}, 0

    def text_turn(self, who: str, text: str) -> str:
        return f"{self.T0}<|{who}_TOKEN|><|START_TEXT|>{text}<|END_TEXT|>{self.T1}"

    def head(self, x: Ctx) -> str:
        entries = ['\n    {"name": ' + go_json(f.get("name", "")) + ', "description": ' + go_json(f.get("description", "")) + ', "parameters": '
                   + go_json(parameters_schema(f.get("parameters")), spaced=True) + ', "responses": null}' for f in (t.get("function") or {} for t in x.tools)]
        listing = ",\n\n".join(entries) + "\n\n" if entries else "\n\n"
        sys = x.conv.system_text
        return self.text_turn("SYSTEM", (sys + "\n\n\n\n" if sys else "") + "# Available Tools\n```json\n[\n" + listing + "\n]\n```")

    def turn_system(self, t: Turn, x: Ctx) -> str:
        return self.text_turn("SYSTEM", t.content)

    def turn_user(self, t: Turn, x: Ctx) -> str:
        return self.text_turn("USER", t.content)

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        out = f"{self.T0}<|CHATBOT_TOKEN|>"
        thinking = f"<|START_THINKING|>{t.thinking}<|END_THINKING|>" if t.thinking else ""
        if t.calls:
            actions = []
            for (name, args), cid in zip(t.calls, t.call_ids):
                number = str(x.memo["next"])
                x.memo["next"] += 1
                if cid:
                    x.memo["numbers"].setdefault(cid, number)
                actions.append('\n\n    {"tool_call_id": "' + number + '", "tool_name": "' + name + '", "parameters": ' + args_json(args, spaced=True) + "}")
            return out + "\n            \n                " + thinking + "<|START_ACTION|>[" + ",".join(actions) + "\n\n]<|END_ACTION|>" + self.T1
        return out + thinking + "<|START_TEXT|>" + t.content + ("" if t is x.conv.last else "<|END_TEXT|>" + self.T1)

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        items = ['\n    {\n        "tool_call_id": "' + x.memo["numbers"].get(rid, rid) + '",\n        "results": {\n\n            \n            "0": '
                 + go_json({"content": c}, spaced=True) + '\n\n        },\n        "is_error": null\n    }' for (_, c), rid in zip(t.results, t.result_ids)]
        return f"{self.T0}<|SYSTEM_TOKEN|><|START_TOOL_RESULT|>[" + ",".join(items) + "\n\n]<|END_TOOL_RESULT|>" + self.T1

    def cue(self, x: Ctx) -> str:
        if x.conv.continued is not None:
            return ""
        return f"{self.T0}<|CHATBOT_TOKEN|>" + ("<|START_THINKING|>" if think_on(x.think, True) else "<|START_THINKING|><|END_THINKING|>")


# ---------------------------------------------------------------------------------------------------
# GLM
# ---------------------------------------------------------------------------------------------------
def _glm_value(v: Any) -> str:
    return v if isinstance(v, str) else go_json(v, sort=True)


class GLM(Dialect):
    """``[gMASK]<sop>`` then ``<|role|>`` marks with no closing mark.  ``airy`` is the 4.6 spelling (a line break after every
    mark and tag, reasoning only on turns after the last question, ``/nothink`` appended to questions); without it the 4.7
    spelling (no line breaks, reasoning of every stored turn kept, ``</think>`` where a turn has none)."""

    system = "inline"

    def __init__(self, airy: bool):
        self.airy = airy
        self.nl = "\n" if airy else ""

    def prepare(self, x: Ctx) -> None:
        x.memo["question"] = x.conv.last_user(default=0)
        x.memo["off"] = x.think is not None and not think_on(x.think, True)

    def head(self, x: Ctx) -> str:
        out = "[gMASK]<sop>"
        if x.tools:
            out += ("<|system|>\n# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                    "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n")
            out += "".join(go_json(tool_schema(t), spaced=not self.airy) + "\n" for t in x.tools)
            out += "</tools>\n\nFor each function call, output the function name and arguments within the following XML format:\n"
            example = ["<tool_call>{function-name}", "<arg_key>{arg-key-1}</arg_key>", "<arg_value>{arg-value-1}</arg_value>", "<arg_key>{arg-key-2}</arg_key>",
                       "<arg_value>{arg-value-2}</arg_value>", "...", "</tool_call>"]
            out += self.nl.join(example)
        return out

    def turn_system(self, t: Turn, x: Ctx) -> str:
        return "<|system|>" + self.nl + t.content

    def turn_user(self, t: Turn, x: Ctx) -> str:
        nudge = "/nothink" if self.airy and x.memo["off"] and not t.content.endswith("/nothink") else ""
        return "<|user|>" + self.nl + t.content + nudge

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        out = "<|assistant|>"
        if self.airy:
            if t.pos > x.memo["question"]:
                out += f"\n<think>{t.thinking}</think>"
        else:
            out += f"<think>{t.thinking}</think>" if t.thinking else "</think>"
        if t.content:
            out += self.nl + t.content
        for name, args in t.calls:
            pairs = "".join(f"<arg_key>{k}</arg_key>{self.nl}<arg_value>{_glm_value(v)}</arg_value>{self.nl}" for k, v in args.items())
            out += f"{self.nl}<tool_call>{name}{self.nl}{pairs}</tool_call>"
        return out

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return "<|observation|>" + "".join(f"{self.nl}<tool_response>{self.nl}{c}{self.nl}</tool_response>" for _, c in t.results)

    def cue(self, x: Ctx) -> str:
        if self.airy:
            return "<|assistant|>" + ("\n<think></think>\n" if x.memo["off"] else "")
        return "<|assistant|>" + ("</think>" if x.memo["off"] else "<think>")


class GLMOcr(GLM):
    """The OCR checkpoints' spelling (model/renderers/glmocr.go:27-107): the 4.7 tool preamble, a line break after every role mark
    and after every stored assistant turn, a ``<think>`` block on every assistant turn (empty when it carries no reasoning),
    ``/nothink`` on questions and an empty block in the cue when reasoning was switched off explicitly, ``[img-N]`` marks in
    front of the text of messages that carry images."""

    def __init__(self, image_tags: bool = True):
        super().__init__(airy=False)
        self.image_tags = image_tags

    def text(self, t: Turn) -> str:
        return image_tagged(t.content, t.images, t.first_image) if self.image_tags else t.content

    def turn_system(self, t: Turn, x: Ctx) -> str:
        return "<|system|>\n" + t.content + "\n"

    def turn_user(self, t: Turn, x: Ctx) -> str:
        nudge = "/nothink" if x.memo["off"] and not t.content.endswith("/nothink") else ""
        return "<|user|>\n" + self.text(t) + nudge

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        out = "<|assistant|>\n<think>" + t.thinking.strip() + "</think>"
        if t.content:
            out += "\n" + t.content.strip()
        for name, args in t.calls:
            out += f"\n<tool_call>{name}" + "".join(f"<arg_key>{k}</arg_key><arg_value>{_glm_value(v)}</arg_value>" for k, v in args.items()) + "</tool_call>"
        return out + "\n"

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return "<|observation|>" + "".join(f"\n<tool_response>\n{c}\n</tool_response>\n" for _, c in t.results)

    def cue(self, x: Ctx) -> str:
        return "<|assistant|>\n" + ("<think></think>\n" if x.memo["off"] else "")


# ---------------------------------------------------------------------------------------------------
# FunctionGemma
# ---------------------------------------------------------------------------------------------------
_ESC = "<escape>"


def _fg(v: Any) -> str:
    """A value in the ``call:`` notation: strings between escape marks, maps with sorted keys, no quotes anywhere."""
    if isinstance(v, str):
        return _ESC + v + _ESC
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, float) and v == int(v):
        return str(int(v))
    if isinstance(v, dict):
        return "{" + ",".join(f"{k}:{_fg(v[k])}" for k in sorted(v)) + "}"
    if isinstance(v, list):
        return "[" + ",".join(map(_fg, v)) + "]"
    return str(v)


class FunctionGemma(Dialect):
    """Gemma turns.  Declarations go into a developer turn; a call and the results that answer it stay inside one model
    turn (``<start_function_call>..<end_function_call><start_function_response>..<end_function_response>``), and the model
    goes on speaking in that same turn after the last result."""

    lead_roles = ("system", "developer")
    bos = "<bos>"
    intro = "You can do function calling with the following functions:"

    def head(self, x: Ctx) -> str:
        sys = x.conv.system_text or ""
        if not (sys or x.tools):
            return self.bos
        out = self.bos + "<start_of_turn>developer\n" + sys.strip()
        if x.tools:
            out += ("\n" if sys else "") + (self.intro if sys.strip() != self.intro else "")
        return out + "".join(map(self.declare, x.tools)) + "<end_of_turn>\n"

    @staticmethod
    def declare(tool: dict[str, Any]) -> str:
        f = tool.get("function") or {}
        params = f.get("parameters") or {}
        out = f"<start_function_declaration>declaration:{f.get('name', '')}{{description:{_ESC}{f.get('description', '')}{_ESC}"
        props, ptype = params.get("properties") or {}, params.get("type") or ""
        if props or ptype or "properties" in params:
            items = []
            if props:
                inner = []
                for name in sorted(props):
                    ty = _types(props[name] or {})
                    inner.append(f"{name}:{{description:{_ESC}{(props[name] or {}).get('description', '')}{_ESC}" + (f",type:{_ESC}{ty[0].upper()}{_ESC}" if ty else "") + "}")
                items.append("properties:{" + ",".join(inner) + "}")
            if params.get("required"):
                items.append("required:[" + ",".join(_ESC + r + _ESC for r in params["required"]) + "]")
            if ptype:
                items.append(f"type:{_ESC}{str(ptype).upper()}{_ESC}")
            out += ",parameters:{" + ",".join(items) + "}"
        return out + "}<end_function_declaration>"

    @staticmethod
    def _answered(t: Turn | None) -> bool:
        return t is not None and t.role == "tool"

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        out = "" if self._answered(x.conv.before(t)) else "<start_of_turn>model\n"
        out += t.content.strip()
        out += "".join("<start_function_call>call:" + name + "{" + ",".join(f"{k}:{_fg(args[k])}" for k in sorted(args)) + "}<end_function_call>" for name, args in t.calls)
        return out + ("<start_function_response>" if t.calls and self._answered(x.conv.after(t)) else "<end_of_turn>\n")

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        prev = x.conv.before(t)
        opened = prev is not None and prev.role == "assistant" and bool(prev.calls)      # the call's turn already printed the first mark
        out = ""
        for i, (name, content) in enumerate(t.results):
            out += ("" if opened and i == 0 else "<start_function_response>") + "response:" + name + "{" + _fg(content) + "}<end_function_response>"
        return out

    def turn_other(self, t: Turn, x: Ctx) -> str:
        header = "" if t.role == "user" and self._answered(x.conv.before(t)) else f"<start_of_turn>{t.role}\n"
        return header + t.content.strip() + "<end_of_turn>\n"

    turn_user = turn_other

    def cue(self, x: Ctx) -> str:
        return "" if self._answered(x.conv.last) else "<start_of_turn>model\n"


# ---------------------------------------------------------------------------------------------------
# Nemotron 3 nano
# ---------------------------------------------------------------------------------------------------
def _py_json(v: Any, shape: str = "any") -> str:
    """A schema value the way the checkpoints' template prints it (``tojson`` of a Python object: ``", "`` and ``": "``
    separators).  ``shape`` says what the wire type of the value is (model/renderers/nemotron3nano.go:382-476): "prop" is one
    parameter's schema, printed with its known keys in a fixed order and a one-element type list as a plain string; "props" a
    map of those in the order sent; anything else prints every key, sorted."""
    if shape == "prop" and isinstance(v, dict):
        parts = []
        ty = _types(v)
        for key in ("anyOf", "type", "items", "description", "enum", "properties", "required"):
            val = v.get(key)
            if key == "type":
                if ty:
                    parts.append('"type": ' + _py_json(ty[0] if len(ty) == 1 else ty))
            elif val not in (None, "", [], {}) or (key == "items" and val is not None):
                parts.append(f'"{key}": ' + _py_json(val, {"anyOf": "proplist", "properties": "props"}.get(key, "any")))
        return "{" + ", ".join(parts) + "}"
    if shape == "props" and isinstance(v, dict):
        return "{" + ", ".join(json.dumps(k, ensure_ascii=False) + ": " + _py_json(p, "prop") for k, p in v.items()) + "}"
    if shape == "proplist" and isinstance(v, list):
        return "[" + ", ".join(_py_json(p, "prop") for p in v) + "]"
    if isinstance(v, dict):
        return "{" + ", ".join(json.dumps(k, ensure_ascii=False) + ": " + _py_json(v[k]) for k in sorted(v)) + "}"
    if isinstance(v, (list, tuple)):
        return "[" + ", ".join(_py_json(i) for i in v) + "]"
    if isinstance(v, float) and v.is_integer() and abs(v) < 1e21:
        return str(int(v))
    return json.dumps(v, ensure_ascii=False)


def _py_str(v: Any) -> str:
    """A call argument or schema scalar as the template's ``str()`` prints it: ``True`` / ``False`` / ``None``, containers as JSON."""
    if v is None:
        return "None"
    if isinstance(v, bool):
        return "True" if v else "False"
    if isinstance(v, (dict, list, tuple)):
        return _py_json(v)
    if isinstance(v, float) and v.is_integer() and abs(v) < 1e21:
        return str(int(v))
    return str(v)


def _strip_think_toggles(s: str) -> str:
    """``/think`` and ``/no_think`` switches go once they have been read; a real ``</think>`` tag stays."""
    return s.replace("</think>", "\0").replace("/think", "").replace("/no_think", "").replace("\0", "</think>")


class Nemotron3Nano(ChatML):
    """ChatML with a system block on every prompt, XML tool declarations and calls in the Qwen3-Coder shape, and a ``<think>``
    block on every assistant turn: the stored reasoning for turns after the last question, an empty pair for earlier ones and
    for answers without reasoning (model/renderers/nemotron3nano.go:23-131).  The 3 checkpoints read ``/think`` and
    ``/no_think`` switches out of system and user text (the last one wins over the request) and delete them; the 3.5
    checkpoints leave text alone, close the reasoning block without line breaks, and ask for short reasoning with a note
    behind the last question when the request's think value is "medium"."""

    def __init__(self, v35: bool = False, image_tags: bool = True):
        self.v35, self.image_tags = v35, image_tags

    def prepare(self, x: Ctx) -> None:
        on = x.think is None or bool(x.think)
        if not self.v35:
            texts = ([x.conv.system_text] if x.conv.system_text is not None else []) + [t.content for t in x.conv.turns if t.role in ("user", "system")]
            for c in texts:
                if "/think" in c.replace("</think>", ""):
                    on = True
                elif "/no_think" in c:
                    on = False
        x.memo["thinking"] = on
        x.memo["question"] = x.conv.last_user()
        x.memo["brief"] = self.v35 and x.think == "medium"

    def head(self, x: Ctx) -> str:
        body = x.conv.system_text or ""
        if not self.v35:
            body = _strip_think_toggles(body)
        if x.tools:
            body += ("\n\n" if body else "") + "# Tools\n\nYou have access to the following functions:\n\n<tools>"
            body += "".join(map(self.declare, x.tools)) + "\n</tools>" + _QWEN3_CODER_CALL_FORMAT
        return self.block("system", body)

    @staticmethod
    def declare(tool: dict[str, Any]) -> str:
        f = tool.get("function") or {}
        params = f.get("parameters") or {}
        out = f"\n<function>\n<name>{f.get('name', '')}</name>"
        if f.get("description"):
            out += f"\n<description>{f['description'].strip()}</description>"
        out += "\n<parameters>"
        for name, prop in (params.get("properties") or {}).items():
            prop = prop if isinstance(prop, dict) else {}
            ty = _types(prop)
            out += f"\n<parameter>\n<name>{name}</name>"
            if ty:
                out += "\n<type>" + (ty[0] if len(ty) == 1 else "[" + ", ".join(f"'{t}'" for t in ty) + "]") + "</type>"
            if prop.get("description"):
                out += f"\n<description>{prop['description'].strip()}</description>"
            if prop.get("enum"):
                out += f"\n<enum>{_py_json(prop['enum'])}</enum>"
            if prop.get("anyOf"):
                out += f"\n<anyOf>{_py_json(prop['anyOf'], 'proplist')}</anyOf>"
            if prop.get("items") is not None:
                out += f"\n<items>{_py_json(prop['items'])}</items>"
            if prop.get("properties") is not None:
                out += f"\n<properties>{_py_json(prop['properties'], 'props')}</properties>"
            if prop.get("required"):
                out += f"\n<required>{_py_json(prop['required'])}</required>"
            out += "\n</parameter>"
        if params.get("$defs") is not None:
            out += f"\n<$defs>{_py_str(params['$defs'])}</$defs>"
        if params.get("items") is not None:
            out += f"\n<items>{_py_str(params['items'])}</items>"
        if params.get("required"):
            out += f"\n<required>{_py_json(params['required'])}</required>"
        return out + "\n</parameters>\n</function>"

    def text(self, t: Turn) -> str:
        return image_tagged(t.content, t.images, t.first_image) if self.image_tags else t.content

    def turn_other(self, t: Turn, x: Ctx) -> str:
        if t.role not in ("user", "system"):
            return self.block(t.role, t.content)
        body = self.text(t)
        if not self.v35:
            body = _strip_think_toggles(body).strip()
        elif t.role == "user" and t.pos == x.memo["question"] and x.memo["brief"]:
            body += "\n\n{reasoning effort: efficient}"
        return self.block(t.role, body)

    turn_user = turn_other

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        # a result with nothing in front of it opens no user block
        return (f"{self.opener}user\n" if t.pos > 0 else "") + "".join(f"<tool_response>\n{c}\n</tool_response>\n" for _, c in t.results) + self.closer

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        body = t.content
        if t.thinking:
            body = "<think>\n" + t.thinking + ("</think>" if self.v35 else "\n</think>\n") + body
        elif "<think>" not in body and "</think>" not in body:
            body = "<think></think>" + body
        earlier = t.pos < x.memo["question"]
        if not t.calls:
            if earlier and "<think>" in body and "</think>" in body:
                body = "<think></think>" + body.rsplit("</think>", 1)[1]
            return self.block("assistant", body.strip())
        if not body.strip():
            body = "<think></think>"
        elif not earlier:
            body = body.strip() + "\n"
        else:
            if "</think>" in body:
                body = body.rsplit("</think>", 1)[1]
            elif "<think>" in body:
                body = body.split("<think>", 1)[0]
            body = ("<think></think>" + body.strip()).strip() + "\n"
        for name, args in t.calls:
            body += f"<tool_call>\n<function={name}>\n" + "".join(f"<parameter={k}>\n{_py_str(v)}\n</parameter>\n" for k, v in args.items())
            body += "</function>\n</tool_call>\n"
        return self.block("assistant", body)

    def cue(self, x: Ctx) -> str:
        return f"{self.opener}assistant\n" + ("<think>\n" if x.memo["thinking"] else "<think></think>")


# ---------------------------------------------------------------------------------------------------
# Laguna (Poolside)
# ---------------------------------------------------------------------------------------------------
_LAGUNA_IDENTITY = ("You are a helpful, conversationally-fluent assistant made by Poolside. You are here to be helpful to users through "
                    "natural language conversations.")
_LAGUNA_CALL_SHAPE = ("For each function call, return an unescaped XML-like object with function name and arguments within '<tool_call>' and "
                      "'</tool_call>' tags, like here:\n")


def _laguna_value(v: Any) -> str:
    return v if isinstance(v, str) else go_json(v, spaced=True)


class Laguna(Dialect):
    """``<role>`` ... ``</role>`` blocks behind the end-of-sequence mark; a default identity when the conversation brings no system
    message; tools as JSON lines inside ``<available_tools>``; every assistant turn opens with its reasoning block or a bare
    closing tag; calls as ``<tool_call>name`` with ``<arg_key>`` / ``<arg_value>`` pairs (model/renderers/laguna.go:24-147).
    ``compact`` is the later checkpoints' spelling (model/renderers/laguna.go:171-262): no line breaks inside blocks, no call
    instructions, stored reasoning printed only when the request reasons, and the trailing assistant turn is closed too."""

    bos = "〈|EOS|〉"

    def __init__(self, compact: bool = False):
        self.compact = compact

    def prepare(self, x: Ctx) -> None:
        x.memo["thinking"] = x.think is not None and bool(x.think)

    def head(self, x: Ctx) -> str:
        system = _LAGUNA_IDENTITY if x.conv.system_text is None else x.conv.system_text
        on, nl = x.memo["thinking"], "" if self.compact else "\n"
        out = self.bos
        if not (system.strip() or x.tools or (self.compact and on)):
            return out
        out += "<system>" + nl
        if system.strip():
            out += nl + system.rstrip()
        if x.tools:
            if not self.compact or system.strip():
                out += "\n\n"
            out += ("### Tools\n\nYou may call functions to assist with the user query.\nAll available function signatures are listed below:\n"
                    "<available_tools>\n" + "".join(go_json(tool_schema(t), spaced=True) + "\n" for t in x.tools) + "</available_tools>")
            if not self.compact:
                out += "\n\n"
                if on:
                    out += "Wrap your thinking in '<think>', '</think>' tags, followed by a function call. " + _LAGUNA_CALL_SHAPE + "<think> your thoughts here </think>\n"
                else:
                    out += _LAGUNA_CALL_SHAPE
                out += "<tool_call>function-name\n<arg_key>argument-key</arg_key>\n<arg_value>value-of-argument-key</arg_value>\n</tool_call>"
        return out + nl + "</system>\n"

    def wrap(self, role: str, body: str) -> str:
        nl = "" if self.compact else "\n"
        return f"<{role}>{nl}{body}{nl}</{role}>\n"

    def turn_user(self, t: Turn, x: Ctx) -> str:
        return self.wrap("user", t.content)

    def turn_system(self, t: Turn, x: Ctx) -> str:
        return self.wrap("system", t.content)

    def turn_tool(self, t: Turn, x: Ctx) -> str:
        return "".join(self.wrap("tool_response", c) for _, c in t.results)

    def turn_assistant(self, t: Turn, x: Ctx) -> str:
        nl = "" if self.compact else "\n"
        calls = "".join(f"<tool_call>{name}{nl}" + "".join(f"<arg_key>{k}</arg_key>{nl}<arg_value>{_laguna_value(v)}</arg_value>{nl}" for k, v in args.items())
                        + f"</tool_call>{nl}" for name, args in t.calls)
        if self.compact:
            return "<assistant>" + (f"<think>{t.thinking}</think>" if x.memo["thinking"] else "</think>") + t.content + calls + "</assistant>\n"
        content, reasoning = t.content, t.thinking
        parts = content.split("</think>")
        if len(parts) > 1:                              # reasoning stored inside the content
            if not reasoning:
                before = parts[0].rstrip("\n")
                reasoning = before[before.rfind("<think>") + len("<think>"):].lstrip("\n") if "<think>" in before else before.lstrip("\n")
            content = parts[-1].lstrip("\n")
        out = "<assistant>\n" + (f"<think>\n{reasoning.strip()}\n</think>\n" if reasoning.strip() else "</think>\n")
        if content.strip():
            out += content.strip() + "\n"
        out += calls
        open_end = t is x.conv.last and bool(content.strip() or reasoning.strip() or t.calls)     # the model continues this turn
        return out + ("" if open_end else "</assistant>\n")

    def cue(self, x: Ctx) -> str:
        last = x.conv.last
        if not self.compact and last is not None and last.role == "assistant":
            return ""
        return "<assistant>" + ("" if self.compact else "\n") + ("<think>" if x.memo["thinking"] else "</think>")


# ---------------------------------------------------------------------------------------------------
# Glimmer
# ---------------------------------------------------------------------------------------------------
_GLIMMER_TOOLS_INTRO = """In this environment you have access to a set of tools you can use to answer the user's question.

You can invoke a function by writing a "<atem:function_calls>" block like the following:
<atem:function_calls>
<atem:invoke name="$FUNCTION_NAME">
<atem:parameter name="$PARAMETER_NAME">$PARAMETER_VALUE</atem:parameter>
...
</atem:invoke>
</atem:function_calls>

String and scalar parameters should be specified as is, while lists and objects should use JSON format. Note that spaces for string values are not stripped. The output is not expected to be valid XML and is parsed with regular expressions.
Here are the functions available in JSONSchema format:
// Tool metadata
"""
_GLIMMER_TOOLS_OUTRO = """

Here's an example of how to call a function in the tool set:
(If the tool namespace is not specified, invoke the function directly as `example_function_name` rather than `example_tool_name.example_function_name`)

to=example_tool_name.example_function_name

<atem:function_calls>
<atem:invoke name="example_tool_name.example_function_name">
<atem:parameter name="example_parameter_1">value_1</atem:parameter>
<atem:parameter name="example_parameter_2">This is the value for the second parameter
that can span
"multiple" lines
</atem:parameter>
</atem:invoke>
</atem:function_calls>"""


class Glimmer(Dialect):
    """``<|start|>header<|message|>body`` messages closed by an end-of-turn or (when the same speaker goes on) end-of-message
    mark; the assistant addresses every message: ``to=self`` for reasoning, ``to=<function>`` for a call written as an
    ``<atem:function_calls>`` block, ``to=user`` for the answer (model/renderers/glimmer.go:289-368).  Every system message
    carries the reasoning strength (from the request, unless its text names one), the tool declarations with their name
    spaces, and the list of valid recipients; without a system message a default one with the knowledge cut-off and the
    current date stands in front.  Works on the messages as sent: a tool result is named by its ``tool_name``, else by the
    call its ``tool_call_id`` points to."""

    bos = "<|begin_of_text|>"
    knowledge_cutoff = "2026-01-04"

    def __init__(self, image_tags: bool = True, current_date: str = ""):
        self.image_tags, self.current_date = image_tags, current_date

    @staticmethod
    def _json(v: Any) -> str:
        return go_json(v, spaced=True, html=False)

    @staticmethod
    def _msg(header: str, body: str, end: str) -> str:
        return f"<|start|>{header}<|message|>{body}{end}"

    def _system(self, text: str, tools: list[dict[str, Any]], strength: str, default: bool) -> str:
        if default:
            today = self.current_date or datetime.date.today().isoformat()
            text += f"\nKnowledge cutoff: {self.knowledge_cutoff}.\nCurrent date: {today}."
        else:
            for a, b in (("Reasoning effort", "Reasoning strength"), ("Reasoning Effort", "Reasoning Strength"),
                         ("reasoning effort", "reasoning strength"), ("REASONING EFFORT", "REASONING STRENGTH")):
                text = text.replace(a, b)
        if default or "reasoning strength" not in text.lower():
            text += f"\n\nReasoning strength: {strength}."
        spaces = list(dict.fromkeys(((t.get("function") or {}).get("name") or "").split(".", 1)[0] for t in tools))
        if tools:
            text += "\n\n" + _GLIMMER_TOOLS_INTRO + "".join('{"name": ' + self._json(n) + ', "description": ""}\n' for n in spaces) + "// Function schemas"
            for t in tools:
                f = t.get("function") or {}
                text += ('\n{"name": ' + self._json(f.get("name") or "") + ', "description": ' + self._json(f.get("description") or "")
                         + ', "parameters": ' + self._json(parameters_schema(f.get("parameters"))) + "}")
            text += _GLIMMER_TOOLS_OUTRO
        text += '\n\n# Valid recipients: "self"' + "".join(f', "{n}.*"' for n in spaces) + ', "user".'
        return self._msg("system", text, "<|eot|>")

    @staticmethod
    def _atem(name: str, args: dict[str, Any]) -> str:
        out = f'<atem:function_calls>\n<atem:invoke name="{name}">\n'
        for k, v in args.items():
            out += f'<atem:parameter name="{k}">' + (Glimmer._json(v) if isinstance(v, (dict, list)) else _xml_scalar(_plain(v, None))) + "</atem:parameter>\n"
        return out + "</atem:invoke>\n</atem:function_calls>"

    def render(self, messages: list[Message], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
        tools = list(tools or [])
        strength = "high" if think is None or think is True else "none" if not think else str(think)
        out = self.bos
        if not any(m.get("role") == "system" for m in messages):
            out += self._system("You are a helpful AI assistant.", tools, strength, True)
        names = {c.get("id"): (c.get("function") or {}).get("name", "") for m in messages for c in m.get("tool_calls") or [] if c.get("id")}
        seen = 0
        for i, m in enumerate(messages):
            role, n = m.get("role"), len(m.get("images") or [])
            body = m.get("content") or ""
            body = image_tagged(body, n, seen) if self.image_tags else "<|patch|>" * n + body
            seen += n
            if role == "system":
                out += self._system(body, tools, strength, False)
            elif role == "user":
                out += self._msg("user", body, "<|eot|>")
            elif role == "tool":
                cid = m.get("tool_call_id") or ""
                name = m.get("tool_name") or names.get(cid, cid)
                out += self._msg("tool " + name, f'<tool_output name="{name}">\n{body}\n</tool_output>', "<|eot|>")
            elif role == "assistant":
                reasoning, calls = m.get("thinking") or "", m.get("tool_calls") or []
                if reasoning:
                    out += self._msg("assistant to=self", reasoning, "<|eom|>")
                goes_on = i + 1 < len(messages) and messages[i + 1].get("role") == "assistant"
                for j, c in enumerate(calls):
                    f = c.get("function") or {}
                    end = "<|eom|>" if j + 1 < len(calls) or goes_on else "<|eot|>"
                    out += self._msg("assistant to=" + f.get("name", ""), self._atem(f.get("name", ""), f.get("arguments") or {}), end)
                if not calls and (body or not reasoning):
                    out += self._msg("assistant to=user", body, "<|eot|>")
        return out + "<|start|>assistant"

    __call__ = render


# ---------------------------------------------------------------------------------------------------
# Gemma 4
# ---------------------------------------------------------------------------------------------------
_G4Q = '<|"|>'                                      # the string delimiter of the format
_G4_STANDARD = ("description", "type", "properties", "required", "nullable")


def _g4_upper(v: Any) -> list[str]:
    return [v.upper()] if isinstance(v, str) else [t.upper() for t in v if isinstance(t, str)] if isinstance(v, (list, tuple)) else []


def _g4_strs(v: Any) -> list[str]:
    return [x for x in v if isinstance(x, str)] if isinstance(v, (list, tuple)) else []


def _g4_num(v: Any) -> str:
    return str(int(v)) if isinstance(v, float) and v.is_integer() else str(v)


def _g4_value(v: Any, schema: bool = False) -> str:
    """A call argument (keys bare) or a schema value (keys quoted): strings between the format's delimiters, maps sorted."""
    if v is None:
        return "null"
    if isinstance(v, str):
        return _G4Q + v + _G4Q
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return _g4_num(v)
    if isinstance(v, dict):
        return "{" + ",".join(((_G4Q + k + _G4Q) if schema else k) + ":" + _g4_value(v[k], schema) for k in sorted(v)) + "}"
    if isinstance(v, (list, tuple)):
        return "[" + ",".join(_g4_value(i, schema) for i in v) + "]"
    return str(v)


def _g4_typed(prop: dict[str, Any]) -> dict[str, Any]:
    """One declared parameter as the wire type keeps it (type, description, enum, items, properties, required; a union of bare
    types written as ``anyOf`` counts as a type list), with a type list folded into one string the way the checkpoints'
    template prints it (model/renderers/gemma4.go:473-513)."""
    out: dict[str, Any] = {}
    ty = _types(prop) if prop.get("type") else []
    if not ty and prop.get("anyOf"):
        bare = all(isinstance(b, dict) and b.get("type") and not any(b.get(k) for k in ("anyOf", "items", "description", "enum", "properties", "required"))
                   for b in prop["anyOf"])
        if bare:
            ty = list(dict.fromkeys(t for b in prop["anyOf"] for t in _types(b)))
    if ty:
        out["type"] = ty[0] if len(ty) == 1 else "[" + ", ".join(f"'{t.upper()}'" for t in ty) + "]"
    if prop.get("description"):
        out["description"] = prop["description"]
    if prop.get("enum"):
        out["enum"] = prop["enum"]
    if prop.get("items") is not None:
        out["items"] = prop["items"]
    if prop.get("properties") is not None:
        out["properties"] = {k: _g4_typed(v if isinstance(v, dict) else {}) for k, v in prop["properties"].items()}
    if prop.get("required"):
        out["required"] = prop["required"]
    return out


def _g4_type_spec(names: list[str]) -> str:
    return "type:" + (_G4Q + names[0] + _G4Q if len(names) == 1 else "[" + ",".join(_G4Q + n + _G4Q for n in names) + "]")


def _g4_required(v: Any) -> str:
    return "required:[" + ",".join(_G4Q + r + _G4Q for r in _g4_strs(v)) + "]"


def _g4_items(items: dict[str, Any]) -> str:
    parts = []
    for key in sorted(items):
        v = items[key]
        if v is None:
            continue
        if key == "properties":
            parts.append("properties:{" + (_g4_props(v) if isinstance(v, dict) else "") + "}")
        elif key == "required":
            parts.append(_g4_required(v))
        elif key == "type":
            names = _g4_upper(v)
            parts.append(_g4_type_spec(names) if names else "")
        else:
            parts.append(key + ":" + _g4_value(v, schema=True))
    return ",".join(parts)


def _g4_props(props: dict[str, Any]) -> str:
    """Parameters by name, sorted: description, then what the first type calls for (enum of a string, items of an array, nested
    properties and required of an object), nullable, and the type last (model/renderers/gemma4.go:329-450)."""
    out = []
    for name in sorted(props):
        prop = props[name]
        if name in _G4_STANDARD or not isinstance(prop, dict):
            continue
        parts = []
        if isinstance(prop.get("description"), str) and prop["description"]:
            parts.append("description:" + _G4Q + prop["description"] + _G4Q)
        names = _g4_upper(prop.get("type"))
        first = names[0] if names else ""
        if first == "STRING" and isinstance(prop.get("enum"), (list, tuple)) and prop["enum"]:
            parts.append("enum:[" + ",".join(_G4Q + (_g4_num(e) if isinstance(e, (int, float)) and not isinstance(e, bool) else
                                                     ("true" if e else "false") if isinstance(e, bool) else str(e)) + _G4Q for e in prop["enum"]) + "]")
        if first == "ARRAY" and isinstance(prop.get("items"), dict) and prop["items"]:
            parts.append("items:{" + _g4_items(prop["items"]) + "}")
        if prop.get("nullable") is True:
            parts.append("nullable:true")
        if first == "OBJECT":
            nested = prop.get("properties")
            parts.append("properties:{" + _g4_props(nested if isinstance(nested, dict) else prop) + "}")
            if _g4_strs(prop.get("required")):
                parts.append(_g4_required(prop["required"]))
        if names:
            parts.append(_g4_type_spec(names))
        out.append(name + ":{" + ",".join(parts) + "}")
    return ",".join(out)


def _g4_without_channels(text: str) -> str:
    """Stored answers lose their ``<|channel>`` ... ``<channel|>`` stretches; one that never closes takes the rest with it."""
    out = ""
    while True:
        a = text.find("<|channel>")
        if a < 0:
            return (out + text).strip()
        out += text[:a]
        b = text.find("<channel|>", a)
        if b < 0:
            return out.strip()
        text = text[b + len("<channel|>"):]


class Gemma4(Dialect):
    """``<|turn>role`` ... ``<turn|>`` turns behind ``<bos>``; a system turn when there is a system (or developer) message, a
    tool or a request to reason (``<|think|>``); tools as ``<|tool>declaration:name{...}<tool|>`` in a key:value notation with
    its own string delimiter; an assistant turn holds its reasoning (after the last question only) as a ``thought`` channel,
    its calls, and the results that answer them, and a run of assistant messages is one model turn; after results the prompt
    goes on inside that turn instead of opening a new one (model/renderers/gemma4.go:24-147).  ``empty_block``: the large
    checkpoints get an empty thought channel in the cue when reasoning is off."""

    bos = "<bos>"

    def __init__(self, image_tags: bool = True, empty_block: bool = False):
        self.image_tags, self.empty_block = image_tags, empty_block

    @staticmethod
    def declare(tool: dict[str, Any]) -> str:
        f = tool.get("function") or {}
        params = f.get("parameters") or {}
        out = "<|tool>declaration:" + (f.get("name") or "") + "{description:" + _G4Q + (f.get("description") or "") + _G4Q
        props = params.get("properties")
        if props is not None or params.get("type"):
            parts = []
            if props:
                parts.append("properties:{" + _g4_props({k: _g4_typed(v if isinstance(v, dict) else {}) for k, v in props.items()}) + "}")
            if params.get("required"):
                parts.append(_g4_required(params["required"]))
            if params.get("type"):
                parts.append("type:" + _G4Q + str(params["type"]).upper() + _G4Q)
            out += ",parameters:{" + ",".join(parts) + "}"
        return out + "}<tool|>"

    def render(self, messages: list[Message], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
        tools = list(tools or [])
        on = think is not None and bool(think)
        lead = bool(messages) and messages[0].get("role") in ("system", "developer")
        msgs = messages[1:] if lead else messages
        out = self.bos
        if lead or tools or on:
            out += "<|turn>system\n" + ("<|think|>\n" if on else "") + (messages[0].get("content") or "").strip() * lead
            out += "".join(map(self.declare, tools)) + "<turn|>\n"
        question = max((i for i, m in enumerate(msgs) if m.get("role") == "user"), default=-1)
        seen = 0

        def text(m: Message, trim: bool) -> str:
            nonlocal seen
            body, n = m.get("content") or "", len(m.get("images") or [])
            if trim:
                body = body.strip()
            if n and self.image_tags:
                body = image_tagged(body, n, seen)
                seen += n
            return body

        def next_speaker(i: int) -> str:
            return next((m.get("role") or "" for m in msgs[i + 1:] if m.get("role") != "tool"), "")

        last_kind, before = "", ""
        for i, m in enumerate(msgs):
            role = m.get("role") or ""
            if role == "tool":
                continue
            last_kind = ""
            shown = "model" if role == "assistant" else role
            if not (shown == "model" and before == "assistant"):
                out += f"<|turn>{shown}\n"
            if role == "assistant" and m.get("thinking") and i > question:
                out += "<|channel>thought\n" + m["thinking"] + "\n<channel|>"
            calls = m.get("tool_calls") or []
            for c in calls:
                f = c.get("function") or {}
                args = f.get("arguments") or {}
                out += "<|tool_call>call:" + f.get("name", "") + "{" + ",".join(k + ":" + _g4_value(args[k]) for k in sorted(args)) + "}<tool_call|>"
                last_kind = "tool_call"
            answered = False
            if calls:
                for r in msgs[i + 1:]:
                    if r.get("role") != "tool":
                        break
                    name = r.get("tool_name") or "unknown"
                    if r.get("tool_call_id"):
                        name = next(((c.get("function") or {}).get("name", "") for c in calls if c.get("id") == r["tool_call_id"]), name)
                    out += "<|tool_response>response:" + name + "{value:" + _g4_value(text(r, False)) + "}<tool_response|>"
                    answered, last_kind = True, "tool_response"
            has_body = False
            if shown == "model":
                if m.get("content") or m.get("images"):
                    m = dict(m, content=_g4_without_channels(m.get("content") or ""))
                    out += text(m, False)
                    has_body = bool(m["content"].strip() or m.get("images"))
            else:
                out += text(m, True)
                has_body = bool((m.get("content") or "").strip() or m.get("images"))
            nxt = next_speaker(i)
            goes_on = shown == "model" and nxt == "assistant" and (not calls or answered)
            if last_kind == "tool_call" and not answered:
                out += "<|tool_response>"
            elif not goes_on and not (answered and not has_body and nxt == ""):
                out += "<turn|>\n"
            before = role
        if last_kind not in ("tool_response", "tool_call"):
            out += "<|turn>model\n" + ("<|channel>thought\n<channel|>" if self.empty_block and not on else "")
        elif last_kind == "tool_response" and on:
            out += "<|channel>thought\n"
        return out

    __call__ = render


# ---------------------------------------------------------------------------------------------------
# registry
# ---------------------------------------------------------------------------------------------------
DIALECTS: dict[str, Callable[[], Dialect]] = {
    "gemma4": lambda: Gemma4(),
    "gemma4-small": lambda: Gemma4(),
    "gemma4-large": lambda: Gemma4(empty_block=True),
    "glimmer": lambda: Glimmer(),
    "laguna": lambda: Laguna(compact=False),
    "poolside-v1": lambda: Laguna(compact=True),
    "nemotron-3-nano": lambda: Nemotron3Nano(v35=False),
    "nemotron-3.5-nano": lambda: Nemotron3Nano(v35=True),
    "qwen3-coder": Qwen3Coder,
    "qwen3-vl-instruct": lambda: Qwen3VL(thinking=False),
    "qwen3-vl-thinking": lambda: Qwen3VL(thinking=True),
    "qwen3.5": lambda: Qwen35(),
    "qwen3.8": lambda: Qwen35(always_block=True, effort=True),
    "ornith": lambda: Qwen35(always_block=True),
    "cogito": Cogito,
    "deepseek3.1": DeepSeek31,
    "olmo3": lambda: Olmo3(extended=False),
    "olmo3.1": lambda: Olmo3(extended=True),
    "olmo3-think": lambda: Olmo3Think(_OLMO31_IDENTITY),
    "olmo3-32b-think": lambda: Olmo3Think("You are a helpful AI assistant."),
    "glm-4.6": lambda: GLM(airy=True),
    "glm-4.7": lambda: GLM(airy=False),
    "glm-ocr": lambda: GLMOcr(),
    "functiongemma": FunctionGemma,
    "cohere": Cohere,
    "lfm2": lambda: LFM2(thinking=False),
    "lfm2-thinking": lambda: LFM2(thinking=True),
}


def renderer_for(name: str | None) -> Dialect | None:
    make = DIALECTS.get(name or "")
    return make() if make else None
