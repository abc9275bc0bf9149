"""Grammar-constrained decoding: a GBNF parser / matcher and a JSON-schema -> GBNF compiler.

``format: "json"`` maps to a built-in JSON grammar and ``format: {schema}`` to a grammar compiled
from the schema; both are enforced while sampling (the reference forwards ``grammar`` /
``json_schema`` to its engine, llm/llama_server.go:52-73, 1583-1599).  The matcher keeps the set of
possible parse stacks (a pushdown automaton over code points); a token is allowed when all of its
characters can be consumed from at least one stack.  The sampler first draws without the grammar and
only consults it for the drawn token, falling back to a filtered redraw on rejection.
"""
from __future__ import annotations

import json
import re
from typing import Any


class GrammarError(ValueError):
    pass


# element kinds: ("char", set_of_ranges, negated) | ("ref", rule_name)
Element = tuple
Alt = list          # list[Element]
Rules = dict        # name -> list[Alt]


class _GbnfParser:
    def __init__(self, src: str):
        self.s, self.i = src, 0
        self.rules: Rules = {}
        self.n_sub = 0

    def ws(self, newlines: bool = True) -> None:
        while self.i < len(self.s):
            c = self.s[self.i]
            if c == "#":
                while self.i < len(self.s) and self.s[self.i] != "\n":
                    self.i += 1
            elif c in " \t" or (newlines and c in "\r\n"):
                self.i += 1
            else:
                break

    def name(self) -> str:
        m = re.compile(r"[A-Za-z_][A-Za-z0-9_-]*").match(self.s, self.i)
        if not m:
            raise GrammarError(f"expected rule name at {self.i}")
        self.i = m.end()
        return m.group(0)

    def parse(self) -> Rules:
        self.ws()
        while self.i < len(self.s):
            n = self.name()
            self.ws(False)
            if not self.s.startswith("::=", self.i):
                raise GrammarError(f"expected ::= after {n}")
            self.i += 3
            self.ws()
            self.rules[n] = self.alternates(n)
            self.ws()
        if "root" not in self.rules:
            raise GrammarError("grammar has no root rule")
        for alts in self.rules.values():
            for alt in alts:
                for el in alt:
                    if el[0] == "ref" and el[1] not in self.rules:
                        raise GrammarError(f"undefined rule {el[1]}")
        return self.rules

    def alternates(self, owner: str) -> list[Alt]:
        alts = [self.sequence(owner)]
        while True:
            self.ws_inline()
            if self.i < len(self.s) and self.s[self.i] == "|":
                self.i += 1
                self.ws()
                alts.append(self.sequence(owner))
            else:
                return alts

    def ws_inline(self) -> None:
        # a newline ends a rule unless the next non-blank character continues it with '|'
        save = self.i
        self.ws(True)
        if self.i < len(self.s) and self.s[self.i] == "|":
            return
        self.i = save
        self.ws(False)

    def char(self) -> str:
        c = self.s[self.i]
        if c == "\\":
            e = self.s[self.i + 1]
            self.i += 2
            if e == "x":
                v = chr(int(self.s[self.i:self.i + 2], 16)); self.i += 2; return v
            if e == "u":
                v = chr(int(self.s[self.i:self.i + 4], 16)); self.i += 4; return v
            if e == "U":
                v = chr(int(self.s[self.i:self.i + 8], 16)); self.i += 8; return v
            return {"n": "\n", "r": "\r", "t": "\t", "\\": "\\", '"': '"', "[": "[", "]": "]", "-": "-", "^": "^"}.get(e, e)
        self.i += 1
        return c

    def new_rule(self, owner: str, alts: list[Alt]) -> str:
        self.n_sub += 1
        n = f"{owner}_{self.n_sub}"
        self.rules[n] = alts
        return n

    def sequence(self, owner: str) -> Alt:
        seq: Alt = []
        while self.i < len(self.s):
            self.ws(False)
            if self.i >= len(self.s):
                break
            c = self.s[self.i]
            start = len(seq)
            if c == '"':
                self.i += 1
                while self.s[self.i] != '"':
                    ch = self.char()
                    seq.append(("char", ((ord(ch), ord(ch)),), False))
                self.i += 1
            elif c == "[":
                self.i += 1
                neg = self.s[self.i] == "^"
                if neg:
                    self.i += 1
                ranges = []
                while self.s[self.i] != "]":
                    a = self.char()
                    if self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                        self.i += 1
                        b = self.char()
                        ranges.append((ord(a), ord(b)))
                    else:
                        ranges.append((ord(a), ord(a)))
                self.i += 1
                seq.append(("char", tuple(ranges), neg))
            elif c == ".":
                self.i += 1
                seq.append(("char", ((0, 0x10FFFF),), False))
            elif c == "(":
                self.i += 1
                self.ws()
                sub = self.alternates(owner)
                self.ws()
                if self.s[self.i] != ")":
                    raise GrammarError("expected )")
                self.i += 1
                seq.append(("ref", self.new_rule(owner, sub)))
            elif re.match(r"[A-Za-z_]", c):
                save = self.i
                n = self.name()
                self.ws(False)
                if self.s.startswith("::=", self.i):      # start of the next rule
                    self.i = save
                    break
                seq.append(("ref", n))
            else:
                break
            # repetition operators apply to the last item (a literal string counts as one item)
            if self.i < len(self.s) and self.s[self.i] in "*+?{":
                item = seq[start:]
                del seq[start:]
                op = self.s[self.i]
                lo, hi = 0, None
                if op == "{":
                    m = re.compile(r"\{(\d+)(?:(,)(\d*))?\}").match(self.s, self.i)
                    if not m:
                        raise GrammarError("bad repetition")
                    lo = int(m.group(1))
                    hi = lo if not m.group(2) else (int(m.group(3)) if m.group(3) else None)
                    self.i = m.end()
                else:
                    self.i += 1
                    lo, hi = {"*": (0, None), "+": (1, None), "?": (0, 1)}[op]
                seq.extend(self.repeat(owner, item, lo, hi))
        return seq

    def repeat(self, owner: str, item: Alt, lo: int, hi: int | None) -> Alt:
        out: Alt = []
        for _ in range(lo):
            out.extend(item)
        if hi is None:
            r = self.new_rule(owner, [])
            self.rules[r] = [list(item) + [("ref", r)], []]
            out.append(("ref", r))
        else:
            # nested optionals: (item (item (item)?)?)?
            tail: Alt = []
            for _ in range(hi - lo):
                r = self.new_rule(owner, [list(item) + tail, []])
                tail = [("ref", r)]
            out.extend(tail)
        return out


def parse_gbnf(src: str) -> Rules:
    try:
        return _GbnfParser(src).parse()
    except GrammarError:
        raise
    except (ValueError, IndexError, KeyError, RecursionError) as e:       # cut-off escapes, text ending inside a construct
        raise GrammarError(f"malformed grammar: {e}") from None


def _match(el: Element, cp: int) -> bool:
    hit = any(a <= cp <= b for a, b in el[1])
    return hit != el[2]


class GrammarMatcher:
    """Set-of-stacks recogniser.  A stack is a tuple of (rule, alt, position) frames, innermost last."""

    def __init__(self, rules: Rules):
        self.rules = rules
        self.stacks = self._expand({((("root", ai, 0),)) for ai in range(len(rules["root"]))})

    def _expand(self, stacks: set) -> set:
        """Advance every stack until its top points at a terminal (or the stack is empty = accepting)."""
        out, seen, work = set(), set(), list(stacks)
        while work:
            st = work.pop()
            if st in seen:
                continue
            seen.add(st)
            if not st:
                out.add(st)
                continue
            rule, ai, pos = st[-1]
            alt = self.rules[rule][ai]
            if pos >= len(alt):
                work.append(st[:-1])            # frame finished: its parent was already advanced when we descended
                continue
            el = alt[pos]
            if el[0] == "char":
                out.add(st)
            else:
                # a reference in the last position needs no return frame: repetitions (R ::= X R | "") then keep a constant
                # depth, and a repetition whose body can match nothing comes back to a stack already seen instead of
                # growing for ever
                base = st[:-1] if pos + 1 >= len(alt) else st[:-1] + ((rule, ai, pos + 1),)
                if len(base) > 2048:
                    raise GrammarError("grammar nests too deeply (left recursion?)")
                for bi in range(len(self.rules[el[1]])):
                    work.append(base + ((el[1], bi, 0),))
        return out

    def _advance(self, stacks: set, cp: int) -> set:
        nxt = set()
        for st in stacks:
            if not st:
                continue
            rule, ai, pos = st[-1]
            el = self.rules[rule][ai][pos]
            if _match(el, cp):
                nxt.add(st[:-1] + ((rule, ai, pos + 1),))
        return self._expand(nxt) if nxt else nxt

    def accepts(self, text: str) -> bool:
        stacks = self.stacks
        for ch in text:
            stacks = self._advance(stacks, ord(ch))
            if not stacks:
                return False
        return True

    def advance(self, text: str) -> None:
        for ch in text:
            self.stacks = self._advance(self.stacks, ord(ch))
            if not self.stacks:
                raise GrammarError("text does not match the grammar")

    def can_end(self) -> bool:
        return () in self.stacks

    def must_end(self) -> bool:
        return self.stacks == {()}


class Grammar:
    """Binds a matcher to a tokenizer: ``allows(token)``, ``accept(token)``, ``done()``."""

    def __init__(self, src: str, tokenizer: Any):
        self.m = GrammarMatcher(parse_gbnf(src))
        self.tk = tokenizer
        self._text: dict[int, str | None] = {}

    def _piece(self, tok: int) -> str | None:
        t = self._text.get(tok, "")
        if t == "":
            try:
                t = self.tk.token_bytes(tok).decode("utf-8")
            except (UnicodeDecodeError, IndexError):
                t = None                     # partial UTF-8 sequences are not offered under a grammar
            self._text[tok] = t
        return t

    def allows(self, tok: int) -> bool:
        if self.tk.is_eog(tok):
            return self.m.can_end()
        if tok in self.tk.special:
            return False
        p = self._piece(tok)
        return bool(p) and self.m.accepts(p)

    def accept(self, tok: int) -> None:
        if self.tk.is_eog(tok):
            return
        p = self._piece(tok)
        if p:
            self.m.advance(p)

    def done(self) -> bool:
        return self.m.must_end()


JSON_GRAMMAR = r'''
root   ::= ws object
value  ::= object | array | string | number | ("true" | "false" | "null") ws
object ::= "{" ws ( string ":" ws value ("," ws string ":" ws value)* )? "}" ws
array  ::= "[" ws ( value ("," ws value)* )? "]" ws
string ::= "\"" ( [^"\\\x7F\x00-\x1F] | "\\" (["\\/bfnrt] | "u" [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F]) )* "\"" ws
number ::= ("-"? ([0-9] | [1-9] [0-9]*)) ("." [0-9]+)? ([eE] [-+]? [0-9]+)? ws
ws     ::= ([ \t\n] ws)?
'''

_PRIMS = {
    "boolean": '("true" | "false") space',
    "number": '("-"? ([0-9] | [1-9] [0-9]*)) ("." [0-9]+)? ([eE] [-+]? [0-9]+)? space',
    "integer": '("-"? ([0-9] | [1-9] [0-9]*)) space',
    "string": r'''"\"" ( [^"\\\x7F\x00-\x1F] | "\\" (["\\/bfnrt] | "u" [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F]) )* "\"" space''',
    "null": '"null" space',
}


class _SchemaCompiler:
    def __init__(self):
        self.rules: dict[str, str] = {"space": '" "?'}

    def add(self, name: str, body: str) -> str:
        base, k = re.sub(r"[^A-Za-z0-9-]", "-", name) or "r", 0
        n = base
        while n in self.rules and self.rules[n] != body:
            k += 1
            n = f"{base}{k}"
        self.rules[n] = body
        return n

    @staticmethod
    def lit(v: Any) -> str:
        s = json.dumps(v, ensure_ascii=False)
        return '"' + s.replace("\\", "\\\\").replace('"', '\\"') + '"'

    def visit(self, schema: Any, name: str) -> str:
        if not isinstance(schema, dict) or not schema:
            return self.any_value()
        if "const" in schema:
            return self.add(name, self.lit(schema["const"]) + " space")
        if "enum" in schema:
            return self.add(name, "(" + " | ".join(self.lit(v) for v in schema["enum"]) + ") space")
        for key in ("anyOf", "oneOf"):
            if key in schema:
                alts = [self.visit(s, f"{name}-{i}") for i, s in enumerate(schema[key])]
                return self.add(name, " | ".join(alts))
        t = schema.get("type")
        if isinstance(t, list):
            alts = [self.visit({**schema, "type": x}, f"{name}-{x}") for x in t]
            return self.add(name, " | ".join(alts))
        if t == "object" or (t is None and "properties" in schema):
            props = schema.get("properties") or {}
            if not props:
                return self.any_object()
            required = set(schema.get("required") or [])
            parts = []
            for k, sub in props.items():
                vr = self.visit(sub, f"{name}-{k}")
                parts.append((k, self.add(f"{name}-{k}-kv", f'{self.lit(k)} space ":" space {vr}'), k in required))
            body = '"{" space '
            req = [p for p in parts if p[2]]
            opt = [p for p in parts if not p[2]]
            seq = " \",\" space ".join(p[1] for p in req)
            if opt:
                # optional members may follow the required ones, in declaration order
                tail = ""
                for p in reversed(opt):
                    inner = p[1] + (f' ( "," space {tail} )?' if tail else "")
                    tail = inner
                if req:
                    seq += f' ( "," space {tail} )?'
                else:
                    seq = f"( {tail} )?"
            body += seq + ' "}" space'
            return self.add(name, body)
        if t == "array":
            item = self.visit(schema.get("items"), f"{name}-item") if schema.get("items") else self.any_value()
            lo, hi = schema.get("minItems", 0), schema.get("maxItems")
            if lo == 0 and hi is None:
                return self.add(name, f'"[" space ( {item} ( "," space {item} )* )? "]" space')
            rep = f'{item} ( "," space {item} )' + (f"{{{max(lo - 1, 0)},{'' if hi is None else hi - 1}}}")
            return self.add(name, f'"[" space ' + (f"( {rep} )?" if lo == 0 else rep) + ' "]" space')
        if t in _PRIMS:
            return self.add(t, _PRIMS[t])
        return self.any_value()

    def any_value(self) -> str:
        if "value" not in self.rules:
            for k, v in _PRIMS.items():
                self.rules[k] = v
            self.rules["value"] = "object | array | string | number | boolean | null"
            self.rules["object"] = '"{" space ( string ":" space value ( "," space string ":" space value )* )? "}" space'
            self.rules["array"] = '"[" space ( value ( "," space value )* )? "]" space'
        return "value"

    def any_object(self) -> str:
        self.any_value()
        return "object"


def json_schema_to_gbnf(schema: dict[str, Any]) -> str:
    c = _SchemaCompiler()
    root = c.visit(schema, "root-v")
    c.rules["root"] = f"space {root}"
    return "\n".join(f"{k} ::= {v}" for k, v in c.rules.items()) + "\n"


def grammar_for_format(fmt: Any) -> str | None:
    """``format`` field of a request -> grammar text (None = unconstrained)."""
    if fmt is None or fmt == "" or fmt == '""':
        return None
    if isinstance(fmt, str):
        if fmt == "json":
            return JSON_GRAMMAR
        try:
            fmt = json.loads(fmt)
        except ValueError:
            raise GrammarError(f'invalid format: {fmt!r}; expected "json" or a JSON schema') from None
        if fmt == "json":
            return JSON_GRAMMAR
    if isinstance(fmt, dict):
        return json_schema_to_gbnf(fmt)
    raise GrammarError('invalid format: expected "json" or a JSON schema')
