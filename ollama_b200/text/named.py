"""Named chat layouts and their detection from a checkpoint's Jinja chat template.

A GGUF or Hugging Face checkpoint describes its prompt format with a Jinja ``chat_template``; a stored model describes it
with a Go template (Modelfile TEMPLATE).  When a model is created from a bare checkpoint the well-known layouts are
recognised and the model gets the equivalent Go template plus the layout's stop strings, so that ``show --template`` and
clients that only understand Go templates see the same thing as with the reference
(template/template.go:72-92 ``Named``, server/create.go ``detectChatTemplate``).

The library is data: a layout is the wrapping of the three roles and the generation prefix; a handful of layouts that fold the
system prompt into a user turn are spelled out.  :func:`gotemplate` turns a layout into Go-template text.  Detection scores a
Jinja template against every layout by the literal markers it must contain and uses the edit distance to a canonical
rendition (:func:`levenshtein`) to separate layouts that share their markers.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class Layout:
    name: str
    system: str = ""            # wrapping of a system message: text with {c}
    user: str = ""
    assistant_open: str = ""    # before an assistant message's content, also the generation prefix unless `generation` is set
    assistant_close: str = ""   # after a finished assistant message (left out after a message that is being continued)
    generation: str | None = None
    stop: tuple[str, ...] = ()
    markers: tuple[str, ...] = ()          # literal substrings a Jinja rendition of this layout contains
    absent: tuple[str, ...] = ()           # ... and must not contain
    custom: str | None = None              # Go-template text for layouts that are not "one wrapping per role"


def _roles(system: str, user: str, a_open: str, a_close: str, generation: str | None = None) -> dict:
    return dict(system=system, user=user, assistant_open=a_open, assistant_close=a_close, generation=generation)


# system prompt folded into the next user turn: the text is written once, not generated
_LLAMA2 = ("{{ $system := \"\" }}{{ range $i, $_ := .Messages }}{{ $last := eq (len (slice $.Messages $i)) 1 }}"
           "{{ if eq .Role \"system\" }}{{ $system = .Content }}"
           "{{ else if eq .Role \"user\" }}[INST] <<SYS>>{{ if $system }}\n{{ $system }}\n{{ end }}<</SYS>>\n\n{{ .Content }} [/INST]{{ $system = \"\" }}"
           "{{ else if eq .Role \"assistant\" }} {{ .Content }}{{ if not $last }}</s><s>{{ end }}"
           "{{ end }}{{ end }}")
_MISTRAL = ("{{ $system := \"\" }}{{ range $i, $_ := .Messages }}{{ $last := eq (len (slice $.Messages $i)) 1 }}"
            "{{ if eq .Role \"system\" }}{{ $system = .Content }}"
            "{{ else if eq .Role \"user\" }}[INST] {{ if $system }}{{ $system }}\n\n{{ end }}{{ .Content }}[/INST]{{ $system = \"\" }}"
            "{{ else if eq .Role \"assistant\" }} {{ .Content }}{{ if not $last }}</s>{{ end }}"
            "{{ end }}{{ end }}")


def _gemma(sep: str, tail: str) -> str:
    return ("{{ $system := \"\" }}{{ range $i, $_ := .Messages }}{{ $last := eq (len (slice $.Messages $i)) 1 }}"
            "{{ if eq .Role \"system\" }}{{ $system = .Content }}"
            "{{ else if eq .Role \"user\" }}<start_of_turn>user\n{{ if $system }}{{ $system }}" + sep + "{{ end }}{{ .Content }}<end_of_turn>\n"
            "{{ $system = \"\" }}{{ if $last }}<start_of_turn>model\n" + tail + "{{ end }}"
            "{{ else if eq .Role \"assistant\" }}<start_of_turn>model\n{{ .Content }}{{ if not $last }}<end_of_turn>\n{{ end }}"
            "{{ end }}{{ end }}")


LAYOUTS: tuple[Layout, ...] = (
    Layout("chatml", **_roles("<|im_start|>system\n{c}<|im_end|>\n", "<|im_start|>user\n{c}<|im_end|>\n", "<|im_start|>assistant\n", "<|im_end|>\n"),
           stop=("<|im_start|>", "<|im_end|>"), markers=("<|im_start|>",)),
    Layout("llama3-instruct", **_roles("<|start_header_id|>system<|end_header_id|>\n\n{c}<|eot_id|>", "<|start_header_id|>user<|end_header_id|>\n\n{c}<|eot_id|>",
                                       "<|start_header_id|>assistant<|end_header_id|>\n\n", "<|eot_id|>"),
           stop=("<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"), markers=("<|start_header_id|>",)),
    Layout("llama2-chat", custom=_LLAMA2, stop=("[INST]", "[/INST]", "<<SYS>>", "<</SYS>>"), markers=("[INST]", "<<SYS>>")),
    Layout("mistral-instruct", custom=_MISTRAL, stop=("[INST]", "[/INST]"), markers=("[INST]",), absent=("<<SYS>>", "Source:")),
    Layout("gemma-instruct", custom=_gemma("\n", ""), stop=("<start_of_turn>", "<end_of_turn>"), markers=("<start_of_turn>",),
           absent=("first_user_prefix",)),
    Layout("gemma3-instruct", custom=_gemma("\n\n", "\n"), stop=("<end_of_turn>",), markers=("<start_of_turn>", "first_user_prefix")),
    Layout("phi-3", **_roles("<|system|>\n{c}<|end|>\n", "<|user|>\n{c}<|end|>\n", "<|assistant|>\n", "<|end|>\n"),
           stop=("<|end|>", "<|system|>", "<|user|>", "<|assistant|>"), markers=("<|end|>",), absent=("<|im_start|>",)),
    Layout("zephyr", **_roles("<|system|>\n{c}</s>\n", "<|user|>\n{c}</s>\n", "<|assistant|>\n", "</s>\n"),
           stop=("<|system|>", "</s>", "<|user|>", "<|assistant|>"), markers=("<|user|>", "eos_token"), absent=("<|end|>",)),
    Layout("command-r", **_roles("<|START_OF_TURN_TOKEN|><|SYSTEM_TOKEN|>{c}<|END_OF_TURN_TOKEN|>", "<|START_OF_TURN_TOKEN|><|USER_TOKEN|>{c}<|END_OF_TURN_TOKEN|>",
                                 "<|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>", "<|END_OF_TURN_TOKEN|>",
                                 generation="<|END_OF_TURN_TOKEN|><|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>\n"),
           stop=("<|START_OF_TURN_TOKEN|>", "<|END_OF_TURN_TOKEN|>"), markers=("<|START_OF_TURN_TOKEN|>",)),
    Layout("openchat", **_roles("GPT4 Correct System: {c}<|end_of_turn|>", "GPT4 Correct User: {c}<|end_of_turn|>", "GPT4 Correct Assistant:", "<|end_of_turn|>",
                                generation="GPT4 Correct Assistant:"),
           stop=("<|end_of_turn|>",), markers=("GPT4 Correct",)),
    Layout("alpaca", **_roles("{c}\n\n", "### Instruction:\n{c}\n\n", "### Response:\n", "\n\n"),
           stop=("### Instruction:", "### Response"), markers=("### Instruction:",)),
    Layout("magicoder", **_roles("{c}\n\n", "@@ Instruction\n{c}\n\n", "@@ Response\n", "\n\n"),
           stop=("@@ Instruction", "@@ Response"), markers=("@@ Instruction",)),
    Layout("starcoder2-instruct", **_roles("{c}\n\n", "### Instruction\n{c}\n\n", "### Response\n", "<|endoftext|>\n\n"),
           stop=("### Instruction", "### Response", "<|endoftext|>"), markers=("### Instruction\n",), absent=("### Instruction:",)),
    Layout("solar-instruct", **_roles("### System:\n{c}\n\n", "### User:\n{c}\n\n", "### Assistant:\n", "</s>\n\n"),
           stop=("### System:", "### User:", "### Assistant"), markers=("### User:",)),
    Layout("granite-instruct", **_roles("System:\n{c}\n\n", "Question:\n{c}\n\n", "Answer:\n", "\n\n"),
           stop=("System:", "Question:", "Answer:"), markers=("Question:",)),
    Layout("chatqa", **_roles("System: {c}\n\n", "User: {c}\n\n", "Assistant:", "\n\n", generation="Assistant:"),
           stop=("System:", "User:", "Assistant:"), markers=("User: ", "Assistant:"), absent=("Falcon", "GPT4", "USER:")),
    Layout("falcon-instruct", **_roles("System: {c}\n", "User:\n{c}\n", "Falcon:\n", "\n"),
           stop=("User:", "Falcon:"), markers=("Falcon:",)),
    Layout("vicuna", **_roles("{c}\n\n", "USER: {c}\n", "ASSISTANT:", "</s>\n", generation="ASSISTANT:"),
           stop=("USER:", "ASSISTANT:"), markers=("USER:", "ASSISTANT:")),
    Layout("alfred", **_roles("<start_system>{c}<end_message>", "<start_user>{c}<end_message>", "<start_assistant>", "<end_message>"),
           stop=("<start_system>", "<end_message>", "<start_user>", "<start_assistant>"), markers=("<start_user>",)),
    Layout("codellama-70b-instruct", **_roles("Source: system\n\n {c} <step> ", "Source: user\n\n {c} <step> ", "Source: assistant\n\n ", " <step> ",
                                              generation="Source: assistant\nDestination: user\n\n "),
           stop=("Source:", "Destination:", "<step>"), markers=("Source:", "<step>")),
)
BY_NAME = {l.name: l for l in LAYOUTS}


def _lit(s: str) -> str:
    """A layout string as Go-template text: literal apart from the content placeholder."""
    return s.replace("{c}", "{{ .Content }}")


def gotemplate(layout: Layout) -> str:
    """The layout as a Go template over ``.Messages``.

    An assistant message that ends the conversation is being continued: its closing text is left out and no generation
    prefix follows.  The separator between an assistant prefix and its content is the prefix's own trailing white space,
    or one blank for prefixes that end in a colon.
    """
    if layout.custom is not None:
        return layout.custom
    a_open = layout.assistant_open
    glue = " " if a_open.endswith(":") else ""
    gen = layout.generation if layout.generation is not None else a_open
    return ("{{ range $i, $_ := .Messages }}{{ $last := eq (len (slice $.Messages $i)) 1 }}"
            "{{ if eq .Role \"system\" }}" + _lit(layout.system) +
            "{{ else if eq .Role \"user\" }}" + _lit(layout.user) + "{{ if $last }}" + gen + "{{ end }}"
            "{{ else if eq .Role \"assistant\" }}" + a_open + glue + "{{ .Content }}{{ if not $last }}" + layout.assistant_close + "{{ end }}"
            "{{ end }}{{ end }}")


def _canonical_jinja(layout: Layout) -> str:
    """A plain Jinja rendition of the layout, used as the reference point of the edit distance."""
    if layout.custom is not None:
        return " ".join(layout.markers)
    def j(s: str) -> str:
        return "{{ '" + s.replace("\n", "\\n").replace("{c}", "' + message['content'] + '") + "' }}"
    return ("{% for message in messages %}{% if message['role'] == 'system' %}" + j(layout.system) + "{% elif message['role'] == 'user' %}" + j(layout.user) +
            "{% else %}" + j(layout.assistant_open + "{c}" + layout.assistant_close) + "{% endif %}{% endfor %}{% if add_generation_prompt %}" +
            j(layout.generation if layout.generation is not None else layout.assistant_open) + "{% endif %}")


def levenshtein(a: str, b: str, limit: int | None = None) -> int:
    """Edit distance (insert / delete / substitute, unit costs).  With ``limit`` the search stops early and returns limit + 1 once
    the distance is known to exceed it."""
    if a == b:
        return 0
    if len(a) < len(b):
        a, b = b, a
    if limit is not None and len(a) - len(b) > limit:
        return limit + 1
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i] + [0] * len(b)
        best = i
        for j, cb in enumerate(b, 1):
            v = prev[j - 1] + (ca != cb)
            if prev[j] + 1 < v:
                v = prev[j] + 1
            if cur[j - 1] + 1 < v:
                v = cur[j - 1] + 1
            cur[j] = v
            if v < best:
                best = v
        if limit is not None and best > limit:
            return limit + 1
        prev = cur
    return prev[-1]


def detect(jinja: str) -> Layout | None:
    """The named layout a Jinja chat template describes, or None.

    A layout is a candidate when the template contains all of its markers and none of the excluded ones; among several
    candidates the one with the most specific markers wins, and the edit distance to the canonical rendition breaks ties.
    """
    if not jinja:
        return None
    text = jinja.replace("\\n", "\n")
    cands = [l for l in LAYOUTS if all(m in text for m in l.markers) and not any(x in text for x in l.absent)]
    if not cands:
        return None
    top = max(sum(len(m) for m in l.markers) for l in cands)
    cands = [l for l in cands if sum(len(m) for m in l.markers) == top]
    if len(cands) == 1:
        return cands[0]
    return min(cands, key=lambda l: levenshtein(jinja, _canonical_jinja(l), 4000))


def named(name: str) -> tuple[str, tuple[str, ...]]:
    """(Go-template text, stop strings) of a layout by name."""
    l = BY_NAME[name]
    return gotemplate(l), l.stop
