"""An interpreter for the subset of Go ``text/template`` that Modelfile TEMPLATEs use.

Supported: text, ``{{- -}}`` trim markers, comments, field chains (``.System``, ``$.Messages``,
``$m.Content``), variables (``:=`` / ``=``), pipelines, parentheses, string / number / bool / nil
literals, ``if / else if / else``, ``range`` (with one or two variables, ``else``, ``break``,
``continue``), ``with``, and the functions ``and or not eq ne lt le gt ge len index slice print
printf println json currentDate yesterdayDate toTypeScriptType``.  Missing keys evaluate to the
zero value (``missingkey=zero``), as configured in the reference (template/template.go:144-165;
function table :120-143).
"""
from __future__ import annotations

import datetime
import json
import re
from typing import Any, Callable


class TemplateError(ValueError):
    pass


# ---------------------------------------------------------------------------------------------
# lexer
# ---------------------------------------------------------------------------------------------
_TOKEN = re.compile(r"""
    (?P<ws>\s+)
  | (?P<str>"(?:\\.|[^"\\])*")
  | (?P<raw>`[^`]*`)
  | (?P<char>'(?:\\.|[^'\\])')
  | (?P<num>[+-]?(?:0x[0-9a-fA-F]+|\d+\.?\d*(?:[eE][+-]?\d+)?|\.\d+))
  | (?P<decl>:=)
  | (?P<assign>=)
  | (?P<pipe>\|)
  | (?P<lp>\()
  | (?P<rp>\))
  | (?P<comma>,)
  | (?P<var>\$[A-Za-z0-9_]*(?:\.[A-Za-z_][A-Za-z0-9_]*)*)
  | (?P<field>(?:\.[A-Za-z_][A-Za-z0-9_]*)+)
  | (?P<dot>\.)
  | (?P<ident>[A-Za-z_][A-Za-z0-9_]*)
""", re.X)


def _lex_action(src: str) -> list[tuple[str, str]]:
    out, pos = [], 0
    while pos < len(src):
        m = _TOKEN.match(src, pos)
        if not m:
            raise TemplateError(f"unexpected {src[pos:pos + 10]!r} in action {{{{{src}}}}}")
        pos = m.end()
        kind = m.lastgroup
        if kind != "ws":
            out.append((kind, m.group(0)))
    return out


def _split(src: str) -> list[tuple[str, str]]:
    """Template source -> [("text", s) | ("action", s)] with trim markers applied."""
    parts: list[tuple[str, str]] = []
    pos = 0
    trim_next = False
    while True:
        i = src.find("{{", pos)
        text = src[pos:] if i < 0 else src[pos:i]
        if trim_next:
            text = text.lstrip(" \t\r\n")
        if i < 0:
            if text:
                parts.append(("text", text))
            break
        j = src.find("}}", i + 2)
        if src.startswith("{{/*", i) or src.startswith("{{- /*", i):
            j = src.find("*/", i)
            j = src.find("}}", j) if j >= 0 else -1
        if j < 0:
            raise TemplateError("unclosed action")
        body = src[i + 2:j]
        ltrim = body.startswith("-") and len(body) > 1 and body[1] in " \t\r\n"
        rtrim = body.endswith("-") and len(body) > 1 and body[-2] in " \t\r\n"
        if ltrim:
            body = body[1:]
            text = text.rstrip(" \t\r\n")
        if rtrim:
            body = body[:-1]
        if text:
            parts.append(("text", text))
        body = body.strip()
        if not (body.startswith("/*") and body.endswith("*/")):
            parts.append(("action", body))
        trim_next = rtrim
        pos = j + 2
    return parts


# ---------------------------------------------------------------------------------------------
# AST
# ---------------------------------------------------------------------------------------------
class Node:
    pass


class Text(Node):
    def __init__(self, s):
        self.s = s


class Action(Node):
    def __init__(self, pipe):
        self.pipe = pipe


class If(Node):
    def __init__(self, pipe, body, orelse):
        self.pipe, self.body, self.orelse = pipe, body, orelse


class Range(Node):
    def __init__(self, vars_, pipe, body, orelse):
        self.vars, self.pipe, self.body, self.orelse = vars_, pipe, body, orelse


class With(Node):
    def __init__(self, pipe, body, orelse):
        self.pipe, self.body, self.orelse = pipe, body, orelse


class Break(Node):
    pass


class Continue(Node):
    pass


class Pipe:
    def __init__(self, decl: list[str], is_assign: bool, cmds: list[list[Any]]):
        self.decl, self.is_assign, self.cmds = decl, is_assign, cmds


class _BreakLoop(Exception):
    pass


class _ContinueLoop(Exception):
    pass


def _parse_pipeline(toks: list[tuple[str, str]], start: int = 0, stop_at_rp: bool = False) -> tuple[Pipe, int]:
    decl: list[str] = []
    is_assign = False
    i = start
    # $x := ... | $i, $e := ... | $x = ...
    if i < len(toks) and toks[i][0] == "var" and "." not in toks[i][1]:
        j = i + 1
        names = [toks[i][1]]
        if j < len(toks) and toks[j][0] == "comma" and j + 1 < len(toks) and toks[j + 1][0] == "var":
            names.append(toks[j + 1][1])
            j += 2
        if j < len(toks) and toks[j][0] in ("decl", "assign"):
            decl, is_assign, i = names, toks[j][0] == "assign", j + 1
    cmds: list[list[Any]] = [[]]
    while i < len(toks):
        k, v = toks[i]
        if k == "pipe":
            cmds.append([])
        elif k == "lp":
            sub, i = _parse_pipeline(toks, i + 1, True)
            cmds[-1].append(("sub", sub))
            continue
        elif k == "rp":
            if not stop_at_rp:
                raise TemplateError("unexpected )")
            return Pipe(decl, is_assign, cmds), i + 1
        elif k == "str":
            cmds[-1].append(("lit", json.loads(v)))
        elif k == "raw":
            cmds[-1].append(("lit", v[1:-1]))
        elif k == "char":
            cmds[-1].append(("lit", ord(json.loads('"' + v[1:-1].replace('"', '\\"') + '"'))))
        elif k == "num":
            cmds[-1].append(("lit", int(v, 0) if re.fullmatch(r"[+-]?(0x[0-9a-fA-F]+|\d+)", v) else float(v)))
        elif k == "var":
            name, _, rest = v.partition(".")
            cmds[-1].append(("var", name, rest.split(".") if rest else []))
        elif k == "field":
            cmds[-1].append(("field", v[1:].split(".")))
        elif k == "dot":
            cmds[-1].append(("dot",))
        elif k == "ident":
            if v in ("true", "false"):
                cmds[-1].append(("lit", v == "true"))
            elif v == "nil":
                cmds[-1].append(("lit", None))
            else:
                cmds[-1].append(("func", v))
        else:
            raise TemplateError(f"unexpected token {v!r}")
        i += 1
    if stop_at_rp:
        raise TemplateError("unclosed (")
    return Pipe(decl, is_assign, cmds), i


class _Parser:
    def __init__(self, parts):
        self.parts, self.i = parts, 0

    def block(self, terminators: tuple[str, ...]) -> tuple[list[Node], str, str]:
        nodes: list[Node] = []
        while self.i < len(self.parts):
            kind, s = self.parts[self.i]
            self.i += 1
            if kind == "text":
                nodes.append(Text(s))
                continue
            word = s.split(None, 1)[0] if s else ""
            rest = s[len(word):].strip()
            if word in terminators:
                return nodes, word, rest
            if word == "if":
                nodes.append(self._if(rest))
            elif word == "range":
                toks = _lex_action(rest)
                pipe, _ = _parse_pipeline(toks)
                vars_, pipe.decl = pipe.decl, []
                body, term, _ = self.block(("else", "end"))
                orelse: list[Node] = []
                if term == "else":
                    orelse, _, _ = self.block(("end",))
                nodes.append(Range(vars_, pipe, body, orelse))
            elif word == "with":
                pipe, _ = _parse_pipeline(_lex_action(rest))
                body, term, _ = self.block(("else", "end"))
                orelse = []
                if term == "else":
                    orelse, _, _ = self.block(("end",))
                nodes.append(With(pipe, body, orelse))
            elif word == "break":
                nodes.append(Break())
            elif word == "continue":
                nodes.append(Continue())
            elif word in ("end", "else"):
                raise TemplateError(f"unexpected {{{{{word}}}}}")
            elif word in ("define", "template", "block"):
                raise TemplateError(f"{{{{{word}}}}} is not supported")
            else:
                pipe, _ = _parse_pipeline(_lex_action(s))
                nodes.append(Action(pipe))
        if terminators:
            raise TemplateError("unexpected EOF: missing {{end}}")
        return nodes, "", ""

    def _if(self, cond: str) -> If:
        pipe, _ = _parse_pipeline(_lex_action(cond))
        body, term, rest = self.block(("else", "end"))
        orelse: list[Node] = []
        if term == "else":
            if rest.startswith("if ") or rest.startswith("if("):
                orelse = [self._if(rest[2:].strip())]      # the nested if consumes the shared {{end}}
            else:
                orelse, _, _ = self.block(("end",))
        return If(pipe, body, orelse)


# ---------------------------------------------------------------------------------------------
# evaluation
# ---------------------------------------------------------------------------------------------
def _truth(v: Any) -> bool:
    if v is None:
        return False
    if isinstance(v, (str, list, tuple, dict)):
        return len(v) > 0
    if isinstance(v, bool):
        return v
    if isinstance(v, (int, float)):
        return v != 0
    return True


def _fmt(v: Any) -> str:
    if v is None:
        return "<no value>"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, float):
        return repr(v) if v != int(v) else str(int(v))
    if isinstance(v, (list, dict)) and type(v).__str__ not in (list.__str__, dict.__str__):
        return str(v)                 # values that define their own text form (tool lists, call arguments: JSON)
    if isinstance(v, (list, tuple)):
        return "[" + " ".join(_fmt(x) for x in v) + "]"
    if isinstance(v, dict):
        return "map[" + " ".join(f"{k}:{_fmt(x)}" for k, x in sorted(v.items())) + "]"
    return str(v)


def _field(v: Any, name: str) -> Any:
    if v is None:
        return None
    if isinstance(v, dict):
        if name in v:
            return v[name]
        # wire structs use snake_case keys; templates use Go field names
        snake = re.sub(r"(?<!^)(?=[A-Z])", "_", name).lower()
        found = v.get(snake, v.get(name.lower()))
        if found is None and name[:1].isupper() and type(v) is not dict and callable(getattr(type(v), name, None)):
            return getattr(v, name)()           # a method of a value that models a Go struct (e.g. ToTypeScriptType)
        return found
    if hasattr(v, name):
        a = getattr(v, name)
        return a() if callable(a) else a
    return None


def _go_printf(fmt: str, *args: Any) -> str:
    it = iter(args)

    def sub(m):
        verb = m.group(2)
        if verb == "%":
            return "%"
        a = next(it, None)
        if verb == "v":
            return _fmt(a)
        if verb == "s":
            return _fmt(a)
        if verb == "q":
            return json.dumps(_fmt(a))
        if verb == "d":
            return str(int(a or 0))
        if verb in "fFgGeE":
            return (m.group(1) + verb) % float(a or 0)
        return _fmt(a)

    return re.sub(r"(%[-+ 0#]*\d*(?:\.\d+)?)([vsqdfFgGeE%])", sub, fmt)


def _slice(v, *idx):
    if v is None:
        return None
    a = idx[0] if len(idx) > 0 else 0
    b = idx[1] if len(idx) > 1 else len(v)
    return v[a:b]


def _index(v, *keys):
    for k in keys:
        if v is None:
            return None
        if isinstance(v, dict):
            v = v.get(k)
        else:
            if not isinstance(k, int) or k < 0 or k >= len(v):
                raise TemplateError(f"index out of range: {k}")
            v = v[k]
    return v


def _cmp(a, b) -> int:
    if a is None or b is None:
        return 0 if a is b else 1
    return (a > b) - (a < b)


def _ts_type(v: Any) -> str:
    if not isinstance(v, dict):
        return "any"
    t = v.get("type")
    if isinstance(t, list):
        return " | ".join(_ts_type({**v, "type": x}) for x in t)
    if v.get("enum"):
        return " | ".join(json.dumps(e) for e in v["enum"])
    return {"string": "string", "number": "number", "integer": "number", "boolean": "boolean", "null": "null",
            "array": (_ts_type(v.get("items")) + "[]") if v.get("items") else "any[]", "object": "Record<string, any>"}.get(t, "any")


FUNCS: dict[str, Callable[..., Any]] = {
    "not": lambda a: not _truth(a),
    "eq": lambda a, *bs: any(_cmp(a, b) == 0 for b in bs),
    "ne": lambda a, b: _cmp(a, b) != 0,
    "lt": lambda a, b: _cmp(a, b) < 0,
    "le": lambda a, b: _cmp(a, b) <= 0,
    "gt": lambda a, b: _cmp(a, b) > 0,
    "ge": lambda a, b: _cmp(a, b) >= 0,
    "len": lambda a: 0 if a is None else len(a),
    "index": _index,
    "slice": _slice,
    "print": lambda *a: "".join(_fmt(x) for x in a),
    "println": lambda *a: " ".join(_fmt(x) for x in a) + "\n",
    "printf": _go_printf,
    "json": lambda v: json.dumps(v, separators=(",", ":"), ensure_ascii=False),
    "currentDate": lambda *a: datetime.date.today().isoformat(),
    "yesterdayDate": lambda *a: (datetime.date.today() - datetime.timedelta(days=1)).isoformat(),
    "toTypeScriptType": _ts_type,
}


class GoTemplate:
    def __init__(self, src: str):
        self.src = src
        try:
            self.root, _, _ = _Parser(_split(src)).block(())
        except TemplateError:
            raise
        except (ValueError, IndexError, KeyError, TypeError, RecursionError) as e:      # e.g. a malformed string literal
            raise TemplateError(f"template: {e}") from None

    # -- introspection (thinking / tool tag inference walks the tree) ---------------------------------
    def identifiers(self) -> set[str]:
        """Lower-cased names of every field referenced anywhere (``.Messages`` -> "messages")."""
        out: set[str] = set()

        def pipe(p: Pipe):
            for cmd in p.cmds:
                for op in cmd:
                    if op[0] == "field":
                        out.update(x.lower() for x in op[1])
                    elif op[0] == "var":
                        out.update(x.lower() for x in op[2])
                    elif op[0] == "sub":
                        pipe(op[1])

        def walk(nodes):
            for n in nodes:
                if isinstance(n, Action):
                    pipe(n.pipe)
                elif isinstance(n, (If, With, Range)):
                    pipe(n.pipe)
                    walk(n.body)
                    walk(n.orelse)

        walk(self.root)
        return out

    # -- execution --------------------------------------------------------------------------------------
    def render(self, data: Any, nodes: list[Node] | None = None) -> str:
        out: list[str] = []
        try:
            self._exec(self.root if nodes is None else nodes, data, [{"$": data}], out)
        except TemplateError:
            raise
        except (TypeError, ValueError, IndexError, KeyError, AttributeError, RecursionError) as e:
            # an operation on values of the wrong kind (Go reports these as execution errors of the template)
            raise TemplateError(f"template: error executing: {e}") from None
        return "".join(out)

    def _lookup(self, scopes, name):
        for s in reversed(scopes):
            if name in s:
                return s[name]
        raise TemplateError(f"undefined variable {name}")

    def _assign(self, scopes, name, val):
        for s in reversed(scopes):
            if name in s:
                s[name] = val
                return
        raise TemplateError(f"undefined variable {name}")

    def _operand(self, op, dot, scopes):
        k = op[0]
        if k == "lit":
            return op[1]
        if k == "dot":
            return dot
        if k == "field":
            v = dot
            for f in op[1]:
                v = _field(v, f)
            return v
        if k == "var":
            v = self._lookup(scopes, op[1])
            for f in op[2]:
                v = _field(v, f)
            return v
        if k == "sub":
            return self._pipe(op[1], dot, scopes)
        raise TemplateError(f"bad operand {op}")

    def _command(self, cmd, dot, scopes, piped=None, has_piped=False):
        if not cmd:
            raise TemplateError("empty command")
        head = cmd[0]
        if head[0] == "func":
            name = head[1]
            if name in ("and", "or"):
                args = cmd[1:]
                val = None
                for a in args:
                    val = self._operand(a, dot, scopes)
                    if (name == "and") != _truth(val):
                        return val
                if has_piped:
                    return piped
                return val
            fn = FUNCS.get(name)
            if fn is None:
                raise TemplateError(f'function "{name}" not defined')
            args = [self._operand(a, dot, scopes) for a in cmd[1:]]
            if has_piped:
                args.append(piped)
            return fn(*args)
        if len(cmd) > 1 or has_piped:
            raise TemplateError("can't give arguments to a non-function")
        return self._operand(head, dot, scopes)

    def _pipe(self, p: Pipe, dot, scopes):
        val, first = None, True
        for cmd in p.cmds:
            val = self._command(cmd, dot, scopes, val, not first)
            first = False
        if p.decl:
            if p.is_assign:
                self._assign(scopes, p.decl[0], val)
            else:
                scopes[-1][p.decl[0]] = val
        return val

    def _exec(self, nodes, dot, scopes, out):
        for n in nodes:
            if isinstance(n, Text):
                out.append(n.s)
            elif isinstance(n, Action):
                v = self._pipe(n.pipe, dot, scopes)
                if not n.pipe.decl:
                    out.append("" if v is None else _fmt(v))
            elif isinstance(n, If):
                scopes.append({})
                try:
                    self._exec(n.body if _truth(self._pipe(n.pipe, dot, scopes)) else n.orelse, dot, scopes, out)
                finally:
                    scopes.pop()
            elif isinstance(n, With):
                scopes.append({})
                try:
                    v = self._pipe(n.pipe, dot, scopes)
                    if _truth(v):
                        self._exec(n.body, v, scopes, out)
                    else:
                        self._exec(n.orelse, dot, scopes, out)
                finally:
                    scopes.pop()
            elif isinstance(n, Range):
                seq = self._pipe(n.pipe, dot, scopes)
                items = list(sorted(seq.items())) if isinstance(seq, dict) else list(enumerate(seq or []))
                if isinstance(seq, int) and not isinstance(seq, bool):
                    items = [(i, i) for i in range(seq)]
                if not items:
                    self._exec(n.orelse, dot, scopes, out)
                    continue
                for k, v in items:
                    sc = {}
                    if len(n.vars) == 1:
                        sc[n.vars[0]] = v
                    elif len(n.vars) == 2:
                        sc[n.vars[0]], sc[n.vars[1]] = k, v
                    scopes.append(sc)
                    try:
                        self._exec(n.body, v, scopes, out)
                    except _ContinueLoop:
                        pass
                    except _BreakLoop:
                        scopes.pop()
                        break
                    scopes.pop()
            elif isinstance(n, Break):
                raise _BreakLoop()
            elif isinstance(n, Continue):
                raise _ContinueLoop()
