"""Streaming splitter of ``<think> ... </think>`` style reasoning from visible content.

The output of a reasoning model has at most one reasoning block, and it opens the message.  The splitter therefore
walks through three phases in order - before the block, inside it, after it - and never goes back; each phase drops
the white space it starts with (after the opening tag, after the closing tag) and the only text ever held back is a
suffix that may still grow into the tag the phase is waiting for.  The observable behaviour is that of the reference's
splitter (thinking/parser.go:57-165): white space in front of the opening tag is tolerated, anything else there means
the message has no reasoning block and is passed through untouched, a second block is ordinary content.  The tag pair
is inferred from the prompt template: the text right before / after the place where a template prints ``.Thinking``
(thinking/template.go:62-119), with ``<think>`` / ``</think>`` as the common default.
"""
from __future__ import annotations

import re

BEFORE, INSIDE, AFTER = range(3)


def _pending(text: str, tag: str) -> int:
    """Length of the longest suffix of ``text`` that is a prefix of ``tag`` (0 if none)."""
    return next((n for n in range(min(len(tag), len(text)), 0, -1) if text.endswith(tag[:n])), 0)


class ThinkingParser:
    def __init__(self, opening: str = "<think>", closing: str = "</think>", started: bool = False):
        self.opening, self.closing = opening, closing
        self.phase = INSIDE if started else BEFORE     # ``started``: the prompt already ends with the opening tag
        self.fresh = True                               # the current phase has not seen anything but white space yet
        self.buf = ""

    def add(self, text: str) -> tuple[str, str]:
        """Feed raw model output; returns (thinking, content) that can be emitted now."""
        self.buf += text
        thinking = ""
        if self.phase == BEFORE:
            probe = self.buf.lstrip()
            if probe.startswith(self.opening):
                self.buf, self.phase = probe[len(self.opening):], INSIDE
            elif self.opening.startswith(probe):
                return "", ""                           # white space or a piece of the tag: undecided
            else:
                self.phase, self.fresh = AFTER, False   # no block: the message passes through as it is
        if self.phase == INSIDE:
            if not self._settle():
                return "", ""
            thinking, found, rest = self.buf.partition(self.closing)
            if not found:
                n = _pending(self.buf, self.closing)
                thinking, self.buf = self.buf[:len(self.buf) - n], self.buf[len(self.buf) - n:]
                return thinking, ""
            self.buf, self.phase, self.fresh = rest, AFTER, True
        if not self._settle():
            return thinking, ""
        content, self.buf = self.buf, ""
        return thinking, content

    def _settle(self) -> bool:
        """Drop the white space a phase begins with; False while there is nothing else yet."""
        if self.fresh:
            self.buf = self.buf.lstrip()
            self.fresh = not self.buf
        return not self.fresh


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
