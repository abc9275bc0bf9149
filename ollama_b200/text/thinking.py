"""Streaming splitter of ``<think> ... </think>`` style reasoning from visible content.

A five-state machine (looking for the opening tag -> eating whitespace after it -> thinking ->
eating whitespace after the closing tag -> done) that holds back only what may still become a
tag, as in the reference (thinking/parser.go:8-28 states, :57-165 transitions).  The tag pair is
inferred from the prompt template: the text right before / after the place where a template prints
``.Thinking`` (thinking/template.go:62-119), with ``<think>`` / ``</think>`` as the common default.
"""
from __future__ import annotations

import re

LOOKING, STARTED_WS, THINKING, DONE_WS, DONE = range(5)


def _overlap(s: str, delim: str) -> int:
    for i in range(min(len(delim), len(s)), 0, -1):
        if s.endswith(delim[:i]):
            return i
    return 0


class ThinkingParser:
    def __init__(self, opening: str = "<think>", closing: str = "</think>", started: bool = False):
        self.opening, self.closing = opening, closing
        self.state = STARTED_WS if started else LOOKING   # ``started``: the prompt already ends with the opening tag
        self.acc = ""

    def add(self, content: str) -> tuple[str, str]:
        """Feed raw model output; returns (thinking, content) that can be emitted now."""
        self.acc += content
        think, rest = [], []
        go = True
        while go:
            t, r, go = self._eat()
            think.append(t)
            rest.append(r)
        return "".join(think), "".join(rest)

    def _eat(self) -> tuple[str, str, bool]:
        st = self.state
        if st == LOOKING:
            trimmed = self.acc.lstrip()
            if trimmed.startswith(self.opening):
                after = trimmed[len(self.opening):].lstrip()
                self.acc = after
                self.state = STARTED_WS if after == "" else THINKING
                return "", "", True
            if self.opening.startswith(trimmed):
                return "", "", False          # partial tag or only whitespace so far
            self.state = DONE
            out, self.acc = self.acc, ""
            return "", out, False
        if st == STARTED_WS:
            trimmed = self.acc.lstrip()
            self.acc = ""
            if trimmed == "":
                return "", "", False
            self.state = THINKING
            self.acc = trimmed
            return "", "", True
        if st == THINKING:
            acc = self.acc
            i = acc.find(self.closing)
            if i >= 0:
                thinking, remaining = acc[:i], acc[i + len(self.closing):].lstrip()
                self.acc = ""
                self.state = DONE_WS if remaining == "" else DONE
                return thinking, remaining, False
            n = _overlap(acc, self.closing)
            if n:
                self.acc = acc[len(acc) - n:]
                return acc[:len(acc) - n], "", False
            self.acc = ""
            return acc, "", False
        if st == DONE_WS:
            trimmed = self.acc.lstrip()
            self.acc = ""
            if trimmed:
                self.state = DONE
            return "", trimmed, False
        out, self.acc = self.acc, ""
        return "", out, False


def infer_tags(template_src: str) -> tuple[str, str]:
    """Opening / closing tag around the spot where the template prints ``.Thinking``; ("", "") if none."""
    m = re.search(r"\{\{-?\s*(?:\$?\w*\.)?\.?Thinking\s*-?\}\}", template_src)
    if not m:
        return "", ""
    before = re.sub(r"\{\{.*?\}\}", "\x00", template_src[:m.start()], flags=re.S).split("\x00")[-1].strip()
    after = re.sub(r"\{\{.*?\}\}", "\x00", template_src[m.end():], flags=re.S).split("\x00")[0].strip()
    o = re.findall(r"<[^<>\s]+>", before)
    c = re.findall(r"</?[^<>\s]+>", after)
    return (o[-1] if o else before.split()[-1] if before.split() else ""), (c[0] if c else after.split()[0] if after.split() else "")


def strip_thinking(content: str, opening: str = "<think>", closing: str = "</think>") -> str:
    """Remove a leading reasoning block from a stored assistant turn (history of qwen3 / deepseek-r1 style models)."""
    p = ThinkingParser(opening, closing)
    _, rest = p.add(content)
    return rest
