"""Built-in prompt renderers and output parsers selected by a model's ``renderer`` / ``parser`` configuration
(Modelfile RENDERER / PARSER), for model families whose chat format is not expressed by a template.

The reference keeps one Go type per family (model/renderers/renderer.go:60-120, model/parsers/parsers.go:46-110).
Here all parsers are instances of one streaming state machine over literal tags (:class:`TagStreamParser`)
that differ in their tags and in how the body of a tool call is decoded:

======================  ==========================  ================================================================
name                    reasoning block             tool call
======================  ==========================  ================================================================
``qwen3``               none                        ``<tool_call>{"name": .., "arguments": {..}}</tool_call>``
``qwen3-thinking``      starts inside ``<think>``   same
``qwen3-vl-instruct``   none                        same
``qwen3-vl-thinking``   starts inside ``<think>``   same; a call may cut the reasoning block short
``qwen3.5``, ``ornith``  starts inside ``<think>``   the qwen3-coder form; a call may cut the reasoning block short
``qwen3-coder``         none                        ``<tool_call><function=f><parameter=k>\\nv\\n</parameter></function></tool_call>``
``ministral``           ``[THINK]..[/THINK]``       ``[TOOL_CALLS]name[ARGS]{json}``
``functiongemma``       none                        ``<start_function_call>call:name{k:<escape>v<escape>}<end_function_call>``
``cogito``              on request, no open tag     ``function<sep>name`` + fenced JSON, between call marks inside a calls block
``deepseek3``           on request, no open tag     ``name<sep>{json}`` between call marks inside a calls block
``olmo3``               none                        ``<function_calls>name(k="v", n=1)`` one per line ``</function_calls>``
``olmo3-think``         starts inside ``<think>``   none
``glm-4.6``             ``<think>..</think>``       ``<tool_call>name<arg_key>k</arg_key><arg_value>v</arg_value></tool_call>``
``glm-4.7``             starts inside ``<think>``   same
``lfm2(-thinking)``     ``<think>..</think>``       ``<|tool_call_start|>[name(k='v'), ...]<|tool_call_end|>``
``cohere``              starts inside the block     JSON list of ``{"tool_call_id", "tool_name", "parameters"}`` between action marks
``passthrough``         none                        none
======================  ==========================  ================================================================

``harmony`` is handled by :mod:`ollama_b200.text.harmony`; the renderers by :mod:`ollama_b200.text.renderers`.
"""
from __future__ import annotations

import ast
import io
import json
import keyword
import re
import tokenize
from dataclasses import dataclass
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


@dataclass
class Region:
    """A stretch of output between two marks that is not prose: one tool call, a list of tool calls, or something to drop.

    ``decode`` turns the body into one call, a list of calls, or None (not a call after all: the stretch is given back as
    the text it was).  ``close`` None means the body has no closing mark and ends where ``body_end`` says.  With ``item``
    the calls stand one by one between marks of their own inside the region and are handed out as each one closes.
    ``drop`` regions are swallowed (a model echoing tool results); ``unwrap`` regions lose their marks only and the body
    stays in the content, white space around it included."""
    open: str
    close: str | None = ""
    decode: Callable[[str], Any] | None = None
    body_end: Callable[[str], int] | None = None
    item: tuple[str, str] | None = None
    drop: bool = False
    unwrap: bool = False
    lenient_end: bool = False                       # the stream may end inside the body: decode what is there


class TagStreamParser:
    """Splits a streamed completion into content, reasoning and tool calls.

    ``add(text, done)`` returns ``(content, thinking, calls)`` for what became unambiguous with this chunk: text that
    could still turn out to be the beginning of a mark (and the white space in front of it) is held back until the
    next chunk decides, and everything held is released when ``done`` is true.
    """

    def __init__(self, *, think_open: str = "", think_close: str = "", start_thinking: bool = False, regions: list[Region] | None = None,
                 call_ends_thinking: bool = False, keep_space: bool = False, drop_marks: dict[str, bool] | None = None, trim_start: bool = False,
                 trim_end: bool = False):
        self.think_open, self.think_close = think_open, think_close
        self.regions = [r for r in regions or [] if r.decode is not None or r.drop or r.unwrap]
        self.call_ends_thinking = call_ends_thinking    # a call that opens inside the reasoning block ends the block
        self.keep_space = keep_space                    # reasoning is handed on with the white space it ends in
        self.trim_start = trim_start                    # white space that opens the reasoning block, or a message without one, goes
        self.trim_end = trim_end                        # white space the answer ends in goes when the stream ends
        self.channel = ""                               # text that names the block right after its opening mark ("thought\n"): dropped
        self.reopen = False                             # a reasoning block may open anywhere in the answer, not only in front of it
        self.mute_thinking = False                      # reasoning is parsed but not handed on
        self.drop_marks = dict(drop_marks or {})        # marks that only frame content: removed; True = white space after them goes too
        self.state: Any = "thinking" if start_thinking and think_close else "content"
        self.may_open_think = bool(think_open)          # an explicit opening tag is accepted at the very start only
        self.skip_ws = False                            # white space right after a closed block belongs to the markup
        self.buf = ""

    # -- helpers ------------------------------------------------------------------------------------
    def _first(self, marks: list[str]) -> tuple[int, str] | None:
        return min(((self.buf.find(m), m) for m in marks if m and m in self.buf), default=None)

    def _region(self, mark: str) -> Region | None:
        return next((r for r in self.regions if r.open == mark), None)

    @staticmethod
    def _held(s: str, tags: list[str]) -> int:
        """Characters at the end of ``s`` to keep back: a possible tag prefix and the white space before it."""
        n = max((_overlap(s, t) for t in tags), default=0)
        head = s[:len(s) - n]
        ws = len(head) - len(head.rstrip())
        return n + ws if (n or ws) and tags else 0

    def _flush(self, sink: list[str], marks: list[str], done: bool) -> None:
        keep = 0 if done else self._held(self.buf, marks)
        sink.append(self.buf[:len(self.buf) - keep])
        self.buf = self.buf[len(self.buf) - keep:]

    @staticmethod
    def _calls(decoded: Any) -> list[dict[str, Any]]:
        return decoded if isinstance(decoded, list) else [decoded]

    # -- the machine --------------------------------------------------------------------------------
    def add(self, text: str, done: bool = False) -> tuple[str, str, list[dict[str, Any]]]:
        self.buf += text
        content: list[str] = []
        thinking: list[str] = []
        calls: list[dict[str, Any]] = []
        while True:
            step = self._in_thinking if self.state == "thinking" else self._in_content if self.state == "content" else self._in_region
            if not step(content, thinking, calls, done):
                break
        return "".join(content), "".join(thinking), calls

    def _in_thinking(self, content, thinking, calls, done) -> bool:
        if self.may_open_think and not self.reopen:     # some checkpoints repeat the opening tag although the prompt ended with it
            t = self.buf.lstrip()
            if t.startswith(self.think_open):
                self.buf, self.may_open_think = t[len(self.think_open):], False
                if self.trim_start:
                    self.lead_ws = True
                return True
            if t and not self.think_open.startswith(t):
                self.may_open_think = False
            elif not done:
                return False
        if getattr(self, "lead_ws", False):
            self.buf = self.buf.lstrip()
            if not self.buf:
                return False
            self.lead_ws = False
        if getattr(self, "name_due", False):
            if self.buf.startswith(self.channel):
                self.buf = self.buf[len(self.channel):]
            elif self.channel.startswith(self.buf) and not done:
                return False
            self.name_due = False
        if self.mute_thinking:
            thinking = []                               # a sink nobody reads
        marks = [self.think_close] + ([r.open for r in self.regions] if self.call_ends_thinking else [])
        hit = self._first(marks)
        if hit is None:
            self._flush(thinking, marks, done)
            return False
        i, mark = hit
        thinking.append(self.buf[:i] if self.keep_space and mark == self.think_close else self.buf[:i].rstrip())
        self.buf = self.buf[i + len(mark):]
        if mark == self.think_close:
            self.state, self.skip_ws = "content", True
        else:
            self.state = self._region(mark)
        return True

    def _in_content(self, content, thinking, calls, done) -> bool:
        if self.skip_ws:
            self.buf = self.buf.lstrip()
            if not self.buf:
                return False
            self.skip_ws = False
        marks = [r.open for r in self.regions] + list(self.drop_marks) + ([self.think_open] if self.may_open_think else [])
        hit = self._first(marks)
        if hit is not None and hit[1] in self.drop_marks:
            i, mark = hit
            content.append(self.buf[:i])
            self.buf, self.skip_ws = self.buf[i + len(mark):], self.drop_marks[mark]
            return True
        if hit is None:
            if self.trim_start and self.may_open_think:     # nothing but white space so far: it goes, whatever follows
                t = self.buf.lstrip()
                if not t or (self.think_open.startswith(t) and not done):
                    return False
                self.buf = t
            before = len(content)
            if done and self.trim_end:
                self.buf = self.buf.rstrip()
            self._flush(content, marks, done)
            if "".join(content[before:]).strip() and not self.reopen:
                self.may_open_think = False
            return False
        i, mark = hit
        before = self.buf[:i]
        if mark == self.think_open and self.may_open_think and self._region(mark) is None:
            if before.strip() and not self.reopen:      # a reasoning block only opens the message
                self.may_open_think = False
                return True
            self.buf, self.state, self.may_open_think = self.buf[i + len(mark):], "thinking", self.reopen
            if self.reopen:
                content.append(before.rstrip())
            if self.trim_start:
                self.lead_ws = True
            self.name_due = bool(self.channel)
            return True
        region = self._region(mark)
        content.append(before if region.unwrap else before.rstrip())
        self.buf, self.state, self.may_open_think = self.buf[i + len(mark):], region, False
        return True

    def _in_region(self, content, thinking, calls, done) -> bool:
        r: Region = self.state
        if r.item is not None:
            return self._in_item_region(r, content, calls, done)
        end = -1
        if r.close:
            i = self.buf.find(r.close)
            if i >= 0:
                body, end = self.buf[:i], i + len(r.close)
        elif r.body_end is not None:
            n = r.body_end(self.buf)
            if n >= 0:
                body, end = self.buf[:n], n
        if end < 0:
            if done and r.lenient_end and self.buf and (decoded := r.decode(self.buf)) is not None:
                calls.extend(self._calls(decoded))
                self.buf, self.state = "", "content"
                return False
            if done:                                    # an unterminated call is returned as text, the way it was produced
                if not r.drop:
                    content.append(("" if r.unwrap else r.open) + self.buf)
                self.buf = ""
            return False
        if r.unwrap:
            content.append(body)
        elif not r.drop:
            decoded = r.decode(body)
            if decoded is not None:
                calls.extend(self._calls(decoded))
            else:
                content.append(r.open + self.buf[:end])
        self.buf = self.buf[end:]
        self.state, self.skip_ws = "content", not r.unwrap
        return True

    def _in_item_region(self, r: Region, content, calls, done) -> bool:
        opener, closer = r.item
        i_end, i_item = self.buf.find(r.close), self.buf.find(closer)
        if i_item >= 0 and (i_end < 0 or i_item < i_end):
            start = self.buf.find(opener)
            body = self.buf[start + len(opener):i_item] if 0 <= start < i_item else self.buf[:i_item]
            decoded = r.decode(body)
            if decoded is not None:
                calls.extend(self._calls(decoded))
            self.buf = self.buf[i_item + len(closer):]
            return True
        if i_end >= 0:
            self.buf = self.buf[i_end + len(r.close):]
            self.state, self.skip_ws = "content", True
            return True
        if done:
            self.buf = ""
        return False


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
    """Declared JSON-schema type(s) of one parameter; the members of an ``anyOf`` count together."""
    def names(p: dict[str, Any]) -> list[str]:
        ty = p.get("type", [])
        return [ty] if isinstance(ty, str) else [x for x in ty if isinstance(x, str)]
    for t in tools or []:
        f = t.get("function", {})
        if f.get("name") == fn:
            p = ((f.get("parameters") or {}).get("properties") or {}).get(param)
            if isinstance(p, dict):
                return [n for alt in p["anyOf"] if isinstance(alt, dict) for n in names(alt)] if p.get("anyOf") else names(p)
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


# -- DeepSeek marks: name and JSON arguments on either side of a separator mark -----------------------------------
_DS_SEP = "<｜tool▁sep｜>"


def _deepseek_call(body: str) -> dict[str, Any] | None:
    """``name<sep>{json}``"""
    name, sep, args = body.partition(_DS_SEP)
    try:
        obj = json.loads(args)
    except ValueError:
        return None
    return {"function": {"name": name.strip(), "arguments": obj}} if sep and isinstance(obj, dict) else None


def _cogito_call(body: str) -> dict[str, Any] | None:
    """``function<sep>name`` followed by the arguments in a fenced ``json`` block"""
    m = re.search(re.escape(_DS_SEP) + r"(.*?)\n```json\n(.*?)\n```", body, re.S)
    if m is None:
        return None
    try:
        obj = json.loads(m.group(2))
    except ValueError:
        return None
    return {"function": {"name": m.group(1).strip(), "arguments": obj}} if isinstance(obj, dict) else None


# -- Python-style calls: name(key="value", n=1), one per line ------------------------------------------------------
_KW = "kw__"
_WORDS = {"true": True, "True": True, "false": False, "False": False, "null": None, "None": None, "nil": None}


def _py_value(node: ast.AST, src: str, raw: bool = False) -> Any:
    """Value of an argument expression: literals, lists and maps as written; the JSON and Python spellings of
    true / false / null; anything else (a bare word, an expression) is the text itself."""
    if isinstance(node, ast.Constant) and not isinstance(node.value, (bytes, complex)) and node.value is not Ellipsis:
        if raw and isinstance(node.value, str):         # the text between the quotes as written, escapes untouched
            seg = ast.get_source_segment(src, node) or ""
            if len(seg) >= 2 and seg[0] in "'\"" and seg[-1] == seg[0] and not seg.startswith(seg[0] * 3):
                return seg[1:-1]
        return node.value
    if isinstance(node, ast.Name) and node.id in _WORDS:
        return _WORDS[node.id]
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.USub, ast.UAdd)) and isinstance(node.operand, ast.Constant) \
            and isinstance(node.operand.value, (int, float)) and not isinstance(node.operand.value, bool):
        return -node.operand.value if isinstance(node.op, ast.USub) else node.operand.value
    if isinstance(node, (ast.List, ast.Tuple)):
        return [_py_value(e, src, raw) for e in node.elts]
    if isinstance(node, ast.Dict) and all(k is not None for k in node.keys):
        return {str(_py_value(k, src, raw)): _py_value(v, src, raw) for k, v in zip(node.keys, node.values)}
    return ast.get_source_segment(src, node) or ""


def _free_keywords(line: str) -> str:
    """Argument names that are Python keywords (``from=``, ``class=``) get a prefix, so that the line parses as Python."""
    try:
        toks = list(tokenize.generate_tokens(io.StringIO(line).readline))
    except (tokenize.TokenError, IndentationError, SyntaxError):
        return line
    for i in range(len(toks) - 2, -1, -1):
        t = toks[i]
        if t.type == tokenize.NAME and keyword.iskeyword(t.string) and t.string not in _WORDS and toks[i + 1].string == "=" and t.start[0] == 1:
            line = line[:t.start[1]] + _KW + line[t.start[1]:]
    return line


def _call_node(node: ast.AST, src: str, raw: bool = False) -> dict[str, Any] | None:
    if not isinstance(node, ast.Call) or node.args or any(k.arg is None for k in node.keywords):
        return None
    name = node.func.id if isinstance(node.func, ast.Name) else (ast.get_source_segment(src, node.func) or "")
    if not name:
        return None
    return {"function": {"name": name, "arguments": {k.arg.removeprefix(_KW): _py_value(k.value, src, raw) for k in node.keywords}}}


def _pythonic_calls(body: str) -> list[dict[str, Any]] | None:
    """One call per line."""
    calls = []
    for line in filter(None, map(str.strip, body.splitlines())):
        line = _free_keywords(line)
        try:
            call = _call_node(ast.parse(line, mode="eval").body, line)
        except (SyntaxError, ValueError):
            return None
        if call is None:
            return None
        calls.append(call)
    return calls


def _python_call_list(body: str) -> list[dict[str, Any]] | None:
    """``[f(a='x'), g(n=1)]``, the same without brackets, or a single call; string values keep their escapes as written
    (model/parsers/lfm2.go:377-470).  Call marks that the model repeated inside the body are ignored."""
    for mark in ("<|tool_call_start|>", "<|tool_call_end|>"):
        body = body.replace(mark, "")
    src = _free_keywords(" ".join(body.strip().splitlines()))
    try:
        tree = ast.parse(src, mode="eval").body
    except (SyntaxError, ValueError):
        return None
    nodes = tree.elts if isinstance(tree, (ast.List, ast.Tuple)) else [tree]
    calls = [_call_node(n, src, raw=True) for n in nodes]
    return None if not calls or any(c is None for c in calls) else calls


# -- GLM: name, then <arg_key>/<arg_value> pairs; values typed by the tool's schema --------------------------------
_GLM_MARKS = re.compile(r"(</?arg_(?:key|value)>)")


def _glm_call(tools: list[dict[str, Any]] | None) -> Callable[[str], dict[str, Any] | None]:
    def decode(body: str) -> dict[str, Any] | None:
        head, *rest = _GLM_MARKS.split(body)
        name = head.strip()
        cols: dict[str, list[str]] = {"key": [], "value": []}
        into: list[str] | None = None
        loose = ""                                      # text outside any pair: a key or value whose opening mark the model left out
        for tok in rest:
            if _GLM_MARKS.fullmatch(tok) is None:
                if into is not None:
                    into[-1] += tok
                else:
                    loose = tok
            elif tok.startswith("</"):
                if into is None and loose.strip():
                    cols["key" if "key" in tok else "value"].append(loose.strip("\n"))
                into, loose = None, ""
            else:
                into, loose = cols["key" if "key" in tok else "value"], ""
                into.append("")
        if not name or len(cols["key"]) != len(cols["value"]):
            return None
        args = {k.strip(): typed_value(v, _schema_types(tools, name, k.strip())) for k, v in zip(cols["key"], cols["value"])}
        return {"function": {"name": name, "arguments": args}}
    return decode


# -- Gemma 4: call:name{key:value,...} with strings between <|"|> marks ------------------------------------------------
_G4_STRING = re.compile(r'<\|"\|>(.*?)<\|"\|>', re.S)
_G4_JSON_STRING = re.compile(r'"(?:\\.|[^"\\])*"')
_G4_KEY = re.compile(r'([{,]\s*)([^\W]+)\s*:', re.UNICODE)


def gemma4_args_to_json(text: str) -> str:
    """The format's argument notation as JSON text: delimited strings become JSON strings (whatever they hold), bare keys are
    quoted; numbers, booleans, null, lists and nested maps are JSON already (model/parsers/gemma4.go:394-447)."""
    held: list[str] = []

    def hold(m: re.Match) -> str:
        held.append(json.dumps(m.group(1), ensure_ascii=False) if m.re is _G4_STRING else m.group(0))
        return f"\x00{len(held) - 1}\x00"
    text = _G4_JSON_STRING.sub(hold, _G4_STRING.sub(hold, text))         # strings a model wrote the JSON way stay as they are
    text = _G4_KEY.sub(lambda m: f'{m.group(1)}"{m.group(2)}":', text)
    return re.sub(r"\x00(\d+)\x00", lambda m: held[int(m.group(1))], text)


def _gemma4_call(body: str) -> dict[str, Any] | None:
    if not body.startswith("call:") or "{" not in body:
        return None
    name, _, rest = body[len("call:"):].partition("{")
    try:
        args = json.loads(gemma4_args_to_json("{" + rest))
    except ValueError:
        return None
    return {"function": {"name": name.strip(), "arguments": args}} if isinstance(args, dict) else None


# -- Laguna: GLM-style pairs, a JSON object behind the name line, or a whole JSON call ------------------------------
_LAGUNA_ALIASES = {"read_file": "read", "write_file": "write", "edit_file": "edit", "web_fetch": "webfetch"}


def _laguna_call(tools: list[dict[str, Any]] | None) -> Callable[[str], dict[str, Any] | None]:
    """``name`` + ``<arg_key>`` / ``<arg_value>`` pairs; ``name`` + a JSON object of arguments; or ``{"name", "arguments"}``
    (model/parsers/laguna.go:424-569).  A name the request did not offer is mapped to the offered tool it commonly stands for
    (``read_file`` -> ``read`` ...); a call repeated inside its own body counts once."""
    declared = {(t.get("function") or {}).get("name") for t in tools or []}
    pairs = _glm_call(tools)

    def resolve(name: str) -> str:
        alias = _LAGUNA_ALIASES.get(name)
        return alias if name not in declared and alias in declared else name

    def decode(body: str) -> dict[str, Any] | None:
        body = body.strip()
        while body.startswith("<tool_call>"):
            body = body[len("<tool_call>"):].strip()
        if body.startswith("{"):
            call = _json_call(body)
            if call is None:
                return None
            call["function"]["name"] = resolve(call["function"]["name"])
            return call
        name, _, rest = body.partition("\n")
        if rest.strip().startswith("{"):
            try:
                args = json.loads(rest.strip())
            except ValueError:
                return None
            return {"function": {"name": resolve(name.strip()), "arguments": args}} if isinstance(args, dict) and name.strip() else None
        call = pairs(body)
        if call is not None:
            call["function"]["name"] = resolve(call["function"]["name"])
        return call
    return decode


# -- Cohere: a JSON list of {"tool_call_id", "tool_name", "parameters"} between action marks ----------------------
def _cohere_actions(body: str) -> list[dict[str, Any]]:
    def call(o: Any) -> dict[str, Any] | None:
        if not isinstance(o, dict) or not isinstance(o.get("tool_name"), str):
            return None
        args = o.get("parameters")
        out: dict[str, Any] = {"function": {"name": o["tool_name"], "arguments": args if isinstance(args, dict) else {}}}
        if o.get("tool_call_id") not in (None, ""):
            out["id"] = str(o["tool_call_id"])
        return out

    body = body.strip()
    try:
        whole = json.loads(body) if body else []
        items = whole if isinstance(whole, list) else [whole]
    except ValueError:                          # a damaged list: take every object that still decodes on its own
        items, dec, i = [], json.JSONDecoder(), body.find("{")
        while i >= 0:
            try:
                obj, end = dec.raw_decode(body, i)
                items.append(obj)
                i = body.find("{", end)
            except ValueError:
                i = body.find("{", i + 1)
    return [c for c in map(call, items) if c is not None]


PARSERS = ("qwen3", "qwen3-thinking", "qwen3-coder", "qwen3.5", "ornith", "qwen3-vl-instruct", "qwen3-vl-thinking", "ministral", "functiongemma", "cogito", "deepseek3",
           "olmo3", "olmo3-think", "glm-4.6", "glm-4.7", "glm-ocr", "cohere", "lfm2", "lfm2-thinking", "nemotron-3-nano", "nemotron-3.5-nano",
           "laguna", "poolside-v1", "glimmer", "gemma4", "gemma4-no-thinking", "passthrough")


# ---------------------------------------------------------------------------------------------------
# Glimmer: addressed messages instead of marks inside one message
# ---------------------------------------------------------------------------------------------------
_ATEM_OPEN, _ATEM_CLOSE = "<atem:function_calls>", "</atem:function_calls>"
_ATEM_PARAM = re.compile(r'<atem:parameter name="([^"]*)">(.*?)</atem:parameter>\n?', re.S)


class GlimmerStreamParser:
    """A completion is a run of messages ``[<|start|>assistant] to=<recipient><|message|>body<|eom|>`` (the last one ends in
    ``<|eot|>``; the prompt already holds the first ``<|start|>assistant``).  ``to=self`` is reasoning, ``to=<declared tool>``
    a call written as an ``<atem:function_calls>`` block, anything else the answer (model/parsers/glimmer.go:55-141).  A tool may
    be addressed with its name space repeated (``ns.ns.fn`` for ``ns.fn``); an answer that is nothing but a call block for
    a declared tool counts as the call (the model forgot the address); a call block that does not parse raises ``ValueError``.
    Same ``add(text, done)`` interface as :class:`TagStreamParser`."""

    HEAD, MSG, ENDS = "<|start|>assistant", "<|message|>", ("<|eom|>", "<|eot|>")

    def __init__(self, tools: list[dict[str, Any]] | None = None, think: Any = None):
        self.tools = {((t.get("function") or {}).get("name") or "").strip(): t for t in tools or []}
        self.tools.pop("", None)
        self.emit_thinking = think is None or bool(think)
        self.state, self.recipient, self.buf, self.streamed = "header", "", "", False

    def _resolve(self, name: str) -> str | None:
        if name in self.tools:
            return name
        ns, dot, fn = name.partition(".")
        return fn if dot and fn in self.tools and fn.partition(".")[0] == ns else None

    def _atem(self, body: str, want: str | None) -> dict[str, Any]:
        body = body.strip()
        if not (body.startswith(_ATEM_OPEN) and body.endswith(_ATEM_CLOSE)):
            raise ValueError("missing ATEM function_calls wrapper")
        inv = body[len(_ATEM_OPEN):-len(_ATEM_CLOSE)].strip()
        if not (inv.startswith('<atem:invoke name="') and inv.endswith("</atem:invoke>") and '">' in inv):
            raise ValueError("missing ATEM invoke wrapper")
        name, _, rest = inv[len('<atem:invoke name="'):-len("</atem:invoke>")].partition('">')
        name = name.replace(self.MSG, "")               # a stray message mark inside the name is dropped
        fn = self._resolve(name)
        if fn is None or (want is not None and fn != want):
            raise ValueError(f"Glimmer recipient {want!r} does not match ATEM invoke {name!r}")
        params, args, pos = rest.strip("\n"), {}, 0
        while pos < len(params):
            m = _ATEM_PARAM.match(params, pos)
            if m is None:
                raise ValueError("malformed ATEM parameter")
            args[m.group(1)] = typed_value(m.group(2), _schema_types(list(self.tools.values()), fn, m.group(1)))
            pos = m.end()
        return {"function": {"name": fn, "arguments": args}}

    def _may_be_call(self) -> bool:
        t = self.buf.lstrip(" \t\r\n")
        return bool(self.tools) and not self.streamed and (_ATEM_OPEN.startswith(t) or t.startswith(_ATEM_OPEN))

    def add(self, text: str, done: bool = False) -> tuple[str, str, list[dict[str, Any]]]:
        self.buf += text
        content, thinking, calls = [], [], []
        while True:
            if self.state == "header":
                if self.buf.startswith(self.HEAD):
                    self.buf = self.buf[len(self.HEAD):]
                elif self.buf.startswith("<") and self.HEAD.startswith(self.buf) and not done:
                    break
                i = self.buf.find(self.MSG)
                if i < 0:
                    if done:                             # no message follows: what is left is text
                        content.append(self.buf)
                        self.buf = ""
                    break
                self.recipient = self.buf[:i].strip().removeprefix("to=").strip()
                self.buf = self.buf[i + len(self.MSG):]
                self.state = "thinking" if self.recipient == "self" else "tool" if self._resolve(self.recipient) else "content"
                self.streamed = False
                continue
            hold = self.state == "tool" or (self.state == "content" and self._may_be_call())
            skip = 0                                    # a call block may hold the text of a mark inside a value
            if hold:
                j = self.buf.find(_ATEM_CLOSE)
                skip = j + len(_ATEM_CLOSE) if j >= 0 else len(self.buf)
            ends = [(k, len(m)) for m in self.ENDS if (k := self.buf.find(m, skip)) >= 0]
            nxt = self.buf.find(self.HEAD, skip)        # the next message begins without an end mark
            if nxt >= 0:
                ends.append((nxt, 0))
            if ends or done:
                k, n = min(ends) if ends else (len(self.buf), 0)
                body, self.buf = self.buf[:k], self.buf[k + n:]
                if self.state == "tool":
                    calls.append(self._atem(body, self._resolve(self.recipient)))
                elif self.state == "thinking":
                    if self.emit_thinking:
                        thinking.append(body)
                elif hold and body.strip().startswith(_ATEM_OPEN) and body.strip().endswith(_ATEM_CLOSE):
                    try:
                        calls.append(self._atem(body, None))
                    except ValueError:
                        content.append(body)
                else:
                    content.append(body)
                self.state, self.recipient = "header", ""
                if not ends:
                    break
                continue
            if hold:
                break
            keep = max(_overlap(self.buf, m) for m in self.ENDS + (self.HEAD,))
            out, self.buf = self.buf[:len(self.buf) - keep], self.buf[len(self.buf) - keep:]
            if out:
                if self.state == "thinking":
                    if self.emit_thinking:
                        thinking.append(out)
                else:
                    content.append(out)
                    self.streamed = True
            break
        return "".join(content), "".join(thinking), calls


def parser_for(name: str | None, tools: list[dict[str, Any]] | None = None, think: Any = None,
               prefill: str = "", after_tool: bool = False) -> "TagStreamParser | GlimmerStreamParser | None":
    """Parser named by a model's configuration, or None when the name is not a built-in of this module.

    ``think`` is the request's think value (None = unset); ``prefill`` the content of a trailing assistant message
    that the model continues (a reasoning model then continues the answer, not the reasoning block).
    """
    asked = think is not None and bool(think)                     # reasoning explicitly requested
    fresh = not prefill
    json_call = Region("<tool_call>", "</tool_call>", _json_call)
    if name == "passthrough":
        return TagStreamParser()
    if name in ("qwen3", "qwen3-thinking"):
        thinking = name == "qwen3-thinking" and think is not False and fresh
        return TagStreamParser(think_open="<think>", think_close="</think>", start_thinking=thinking, regions=[json_call] if tools else [])
    if name in ("qwen3-vl-instruct", "qwen3-vl-thinking"):        # model/parsers/qwen3vl.go:50-64: the variant decides, not the request
        thinking = name == "qwen3-vl-thinking" and fresh
        return TagStreamParser(think_close="</think>", start_thinking=thinking, regions=[json_call], call_ends_thinking=True)
    if name == "qwen3-coder":
        return TagStreamParser(regions=[Region("<tool_call>", "</tool_call>", _xml_call(tools))])
    if name in ("qwen3.5", "ornith"):             # model/parsers/qwen35.go:57-78: reasoning unless switched off, XML calls, a call ends the block
        return TagStreamParser(think_open="<think>", think_close="</think>", start_thinking=think is not False and (think is None or bool(think)) and fresh,
                               regions=[Region("<tool_call>", "</tool_call>", _xml_call(tools))], call_ends_thinking=True)
    if name in ("gemma4", "gemma4-no-thinking"):
        # model/parsers/gemma4.go:66-92, :167-365: a thought channel may open anywhere in the answer and is handed on only when the
        # request reasons; after tool results the prompt goes on inside the model's turn, so a reasoning request starts in the
        # channel; what the model adds behind a call (a second closing mark, the mark that opens a result) goes
        asked_now = think is not None and bool(think) and name == "gemma4"      # the other name: checkpoints that never reason
        p = TagStreamParser(think_open="<|channel>", think_close="<channel|>", start_thinking=asked_now and after_tool,
                            drop_marks={"<tool_call|>": True, "<|tool_response>": True},
                            regions=[Region("<|tool_call>", "<tool_call|>", _gemma4_call, lenient_end=True)])
        p.channel, p.reopen, p.mute_thinking = "thought\n", True, not asked_now
        p.may_open_think = True
        return p
    if name == "glimmer":
        return GlimmerStreamParser(tools, think)
    if name in ("laguna", "poolside-v1"):
        # model/parsers/laguna.go:68-95: reasoning only on request; the later checkpoints close a continued turn in the prompt, so
        # they always start fresh.  A closing tag the model repeats (the prompt ends with one when reasoning is off) goes.
        thinking = asked and (fresh or name == "poolside-v1")
        p = TagStreamParser(think_open="<think>", think_close="</think>", start_thinking=thinking, trim_start=True, trim_end=True, call_ends_thinking=True,
                            drop_marks={"</think>": True}, regions=[Region("<tool_call>", "</tool_call>", _laguna_call(tools))])
        p.skip_ws = p.state == "content"
        return p
    if name in ("nemotron-3-nano", "nemotron-3.5-nano"):
        # model/parsers/nemotron3nano.go:46-66: the prompt ends inside the reasoning block unless reasoning is off or an answer is
        # being continued; a repeated opening tag and the white space behind it go; a call without a closing tag ends the block
        thinking = (think is None or bool(think)) and fresh
        return TagStreamParser(think_open="<think>" if thinking else "", think_close="</think>", start_thinking=thinking, trim_start=thinking,
                               regions=[Region("<tool_call>", "</tool_call>", _xml_call(tools))], call_ends_thinking=True)
    if name == "functiongemma":
        return TagStreamParser(regions=[Region("<start_function_call>", "<end_function_call>", _functiongemma_call)])
    if name == "ministral":
        return TagStreamParser(think_open="[THINK]", think_close="[/THINK]",
                               regions=[Region("[TOOL_CALLS]", None, _ministral_call, body_end=_ministral_end)])
    if name in ("cogito", "deepseek3"):
        # model/parsers/cogito.go:64-87, deepseek3.go:61-78: reasoning only on request; cogito does not reason when tools are offered
        thinking = asked and fresh and not (name == "cogito" and tools)
        one = _cogito_call if name == "cogito" else _deepseek_call
        calls = Region("<｜tool▁calls▁begin｜>", "<｜tool▁calls▁end｜>", one, item=("<｜tool▁call▁begin｜>", "<｜tool▁call▁end｜>"))
        echo = (Region("<｜tool▁outputs▁begin｜>", "<｜tool▁outputs▁end｜>", drop=True) if name == "cogito"
                else Region("<｜tool▁output▁begin｜>", "<｜tool▁output▁end｜>", unwrap=True))
        return TagStreamParser(think_close="</think>", start_thinking=thinking, regions=[calls, echo])
    if name == "cohere":
        # model/parsers/cohere.go:66-84: the prompt ends inside the reasoning block unless reasoning is off; the answer comes in
        # text (or response) marks, calls in action marks; the marks themselves and the white space between blocks go
        frames = {"<|START_TEXT|>": False, "<|START_RESPONSE|>": False, "<|END_TEXT|>": True, "<|END_RESPONSE|>": True, "<|END_OF_TURN_TOKEN|>": True}
        p = TagStreamParser(think_close="<|END_THINKING|>", start_thinking=(think is None or bool(think)) and fresh, drop_marks=frames,
                            regions=[Region("<|START_ACTION|>", "<|END_ACTION|>", _cohere_actions)])
        p.skip_ws = fresh and p.state == "content"
        return p
    if name in ("lfm2", "lfm2-thinking"):
        # model/parsers/lfm2.go:62-82: a thinking variant that was asked to think may open a block with an explicit tag, or answer directly
        may_think = name == "lfm2-thinking" and asked and fresh
        return TagStreamParser(think_open="<think>" if may_think else "", think_close="</think>" if may_think else "", trim_start=may_think,
                               regions=[Region("<|tool_call_start|>", "<|tool_call_end|>", _python_call_list)])
    if name == "olmo3":
        return TagStreamParser(regions=[Region("<function_calls>", "</function_calls>", _pythonic_calls)])
    if name == "olmo3-think":                                     # model/parsers/olmo3_think.go:43-55: the prompt always ends in <think>
        return TagStreamParser(think_close="</think>", start_thinking=fresh)
    if name == "glm-ocr":                                         # model/parsers/glmocr.go:5-17: the 4.6 parser with reasoning off
        return TagStreamParser(regions=[Region("<tool_call>", "</tool_call>", _glm_call(tools))])
    if name in ("glm-4.6", "glm-4.7"):
        # model/parsers/glm47.go:13-20: the 4.7 prompt ends inside the block unless reasoning was switched off
        thinking = name == "glm-4.7" and (think is None or bool(think))
        return TagStreamParser(think_open="<think>", think_close="</think>", start_thinking=thinking,
                               regions=[Region("<tool_call>", "</tool_call>", _glm_call(tools))])
    return None


# ---------------------------------------------------------------------------------------------------
# renderers live in :mod:`ollama_b200.text.renderers`; the two oldest keep their function names here
# ---------------------------------------------------------------------------------------------------
from .renderers import DIALECTS, renderer_for  # noqa: E402,F401


def render_qwen3_coder(messages: list[dict[str, Any]], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
    return renderer_for("qwen3-coder").render(messages, tools, think)


def render_functiongemma(messages: list[dict[str, Any]], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
    return renderer_for("functiongemma").render(messages, tools, think)
