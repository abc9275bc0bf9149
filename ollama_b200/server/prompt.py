"""Prompt assembly for chat requests.

``chat_prompt`` renders the conversation and, when it does not fit ``num_ctx``, drops the oldest
messages while always keeping the system messages and the latest message (server/prompt.go:23-92).
Rendering precedence (server/routes.go:2357-2385, server/images.go:322-339): a built-in RENDERER, harmony for gpt-oss, the
Modelfile Go TEMPLATE, the GGUF Jinja chat template, otherwise the bare prompt.
"""
from __future__ import annotations

from typing import Any, Callable

from ..text import harmony
from ..text.builtin import renderer_for
from ..text.template import DEFAULT_TEMPLATE, JinjaChatTemplate, Template


class PromptRenderer:
    """Everything needed to turn messages into a prompt string for one model."""

    def __init__(self, model: Any, tokenizer: Any = None):
        self.model = model
        kv = model.kv() if hasattr(model, "kv") else {}
        self.arch = kv.get("general.architecture", "")
        self.is_harmony = self.arch in ("gpt-oss", "gptoss") and not model.template
        self.go_template = Template(model.template) if model.template else None
        self.jinja = None
        ct = model.chat_template() if hasattr(model, "chat_template") else ""
        if ct and self.go_template is None and not self.is_harmony:
            bos = eos = ""
            if tokenizer is not None:
                bos = tokenizer.tokens[tokenizer.bos] if 0 <= tokenizer.bos < tokenizer.n_vocab else ""
                eos = tokenizer.tokens[tokenizer.eos] if 0 <= tokenizer.eos < tokenizer.n_vocab else ""
            try:
                self.jinja = JinjaChatTemplate(ct, bos, eos)
            except Exception:
                self.jinja = None
        self.names = harmony.FunctionNameMap()
        # a renderer named by the model's configuration (Modelfile RENDERER) takes precedence over its templates
        self.builtin = renderer_for((getattr(model, "config", None) or {}).get("renderer"))

    @property
    def template_source(self) -> str:
        if self.go_template is not None:
            return self.go_template.raw
        return self.jinja.raw if self.jinja is not None else ""

    def render_chat(self, messages: list[dict[str, Any]], tools: list[dict[str, Any]] | None = None, think: Any = None) -> str:
        if self.builtin is not None:
            return self.builtin(messages, tools, think)
        if self.is_harmony:
            return harmony.render_prompt(messages, tools, think, self.names)
        if self.go_template is not None:
            level = think if isinstance(think, str) else ""
            return self.go_template.execute(messages=messages, tools=tools, think=bool(think) if think is not None else False,
                                            think_level=level, is_think_set=think is not None)
        if self.jinja is not None:
            kw: dict[str, Any] = {}
            if think is not None:
                kw["enable_thinking"] = bool(think)
                if isinstance(think, str):
                    kw["reasoning_effort"] = think
            return self.jinja.render(messages, tools, True, **kw)
        return "\n".join(m.get("content", "") for m in messages)

    def render_generate(self, system: str, prompt: str, suffix: str = "", template: str | None = None, think: Any = None) -> str:
        if template:
            t = Template(template)
        elif self.go_template is not None:
            t = self.go_template
        elif self.jinja is not None or self.is_harmony:
            msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": prompt}]
            return self.render_chat(msgs, None, think)
        else:
            t = Template(DEFAULT_TEMPLATE)
        if suffix:
            return t.execute(prompt=prompt, suffix=suffix)
        level = think if isinstance(think, str) else ""
        return t.render_generate(system, prompt, think=bool(think) if think is not None else False, think_level=level,
                                 is_think_set=think is not None)


def chat_prompt(render: Callable[[list[dict[str, Any]]], str], count_tokens: Callable[[str], int], messages: list[dict[str, Any]],
                num_ctx: int, truncate: bool = True) -> tuple[str, list[dict[str, Any]]]:
    """Return (prompt, messages actually used).

    With ``truncate`` the oldest messages are dropped (system messages stay) until the rendered prompt fits ``num_ctx``; the
    last message is always kept.  The walk starts from the whole conversation, so a chat that fits costs one rendering and
    one tokenisation (server/prompt.go:23-92 of the reference)."""
    n = 0
    if truncate:
        last = len(messages) - 1
        for i in range(last + 1):
            cand = [m for m in messages[:i] if m.get("role") == "system"] + messages[i:]
            p = render(cand)
            if count_tokens(p) <= num_ctx:
                return p, cand
            n = i
        n = max(last, 0)
    used = [m for m in messages[:n] if m.get("role") == "system"] + messages[n:]
    return render(used), used
