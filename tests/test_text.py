"""Prompt templates, output parsers, tokenizers and the grammar engine."""
import pytest

from ollama_b200.engine.grammar import JSON_GRAMMAR, Grammar, GrammarError, GrammarMatcher, grammar_for_format, json_schema_to_gbnf, parse_gbnf
from ollama_b200.text import harmony
from ollama_b200.text.gotemplate import GoTemplate, TemplateError
from ollama_b200.text.template import JinjaChatTemplate, Template, collate
from ollama_b200.text.thinking import ThinkingParser, infer_tags, strip_thinking
from ollama_b200.text.tokenizer import BPETokenizer, SPMTokenizer, _byte_to_unicode, tokenizer_from_gguf
from ollama_b200.text.tools import ToolParser, infer_tag

CHATML = """{{- range $i, $_ := .Messages }}{{- $last := eq (len (slice $.Messages $i)) 1 }}<|im_start|>{{ .Role }}
{{ .Content }}{{ if not $last }}<|im_end|>
{{ end }}{{ if and $last (ne .Role "assistant") }}<|im_end|>
<|im_start|>assistant
{{ end }}{{- end }}"""


def test_go_template_language():
    t = GoTemplate('{{ if and .A (not .B) }}x{{ else if .C }}y{{ else }}z{{ end }}|{{ range $i, $v := .L }}{{ $i }}={{ $v }},{{ end }}'
                   '|{{ with .M }}{{ .k }}{{ end }}|{{ printf "%s-%d" .S 7 }}|{{ .Missing }}|{{ len .L }}|{{ index .L 1 }}|{{ json .M }}')
    out = t.render({"A": True, "B": False, "C": True, "L": ["p", "q"], "M": {"k": "v"}, "S": "s"})
    assert out == 'x|0=p,1=q,|v|s-7||2|q|{"k":"v"}'
    assert GoTemplate("a  {{- 1 }}  {{ 2 -}}  b").render({}) == "a1  2b"
    assert GoTemplate("{{/* c */}}x{{ range .L }}{{ if eq . 2 }}{{ break }}{{ end }}{{ . }}{{ end }}").render({"L": [1, 2, 3]}) == "x1"
    assert GoTemplate("{{ $x := 1 }}{{ if true }}{{ $x = 2 }}{{ end }}{{ $x }}").render({}) == "2"
    assert GoTemplate("{{ range .L }}a{{ else }}empty{{ end }}").render({"L": []}) == "empty"
    with pytest.raises(TemplateError):
        GoTemplate("{{ if .A }}x")
    with pytest.raises(TemplateError):
        GoTemplate("{{ nosuchfunc 1 }}").render({})


def test_template_modes_and_collate():
    legacy = Template("{{ if .System }}<|system|>{{ .System }}<|end|>{{ end }}{{ if .Prompt }}<|user|>{{ .Prompt }}<|end|>{{ end }}"
                      "<|assistant|>{{ .Response }}<|end|>")
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
            {"role": "user", "content": "again"}]
    assert legacy.execute(messages=msgs) == "<|system|>S<|end|><|user|>hi<|end|><|assistant|>yo<|end|><|user|>again<|end|><|assistant|>"
    # an assistant message at the end is a prefill: the prompt ends with it
    assert legacy.execute(messages=msgs[:2] + [{"role": "assistant", "content": "par"}]).endswith("<|assistant|>par")
    chat = Template(CHATML)
    assert chat.execute(messages=msgs[1:]) == ("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\nyo<|im_end|>\n"
                                               "<|im_start|>user\nagain<|im_end|>\n<|im_start|>assistant\n")
    assert Template("{{ .Prompt }}").t.src.endswith("{{ .Response }}")      # response slot appended when absent
    assert Template("<PRE> {{ .Prompt }} <SUF>{{ .Suffix }} <MID>").execute(prompt="a", suffix="b") == "<PRE> a <SUF>b <MID>"
    system, merged = collate([{"role": "system", "content": "a"}, {"role": "user", "content": "1"}, {"role": "user", "content": "2"},
                              {"role": "system", "content": "b"}])
    assert system == "a\n\nb" and merged[1]["content"] == "1\n\n2"
    tools = Template("{{ if .Tools }}T:{{ .Tools }}{{ end }}{{ range .Messages }}{{ range .ToolCalls }}[{{ .Function.Name }} {{ .Function.Arguments }}]{{ end }}{{ end }}")
    out = tools.execute(messages=[{"role": "assistant", "tool_calls": [{"function": {"name": "f", "arguments": {"x": 1}}}]}],
                        tools=[{"type": "function", "function": {"name": "f", "parameters": {}}}])
    assert '"name":"f"' in out and '[f {"x":1}]' in out


def test_template_values_of_tools_and_calls_as_in_the_reference():
    """template/template_test.go:455-790 and api/types.go:429-471 of the reference: date helpers, call arguments and tool
    properties print as JSON, both can be ranged over by key, a property knows the TypeScript spelling of its type."""
    import datetime
    import json as js
    from ollama_b200.text.template import Template, collate
    user = [{"role": "user", "content": "Hello"}]
    today = datetime.date.today()
    assert Template("{{- range .Messages }}{{ .Content }}{{ end }} Today is {{ currentDate }}").execute(messages=user) == f"Hello Today is {today.isoformat()}"
    assert Template("{{- range .Messages }}{{ end }}{{ yesterdayDate }}").execute(messages=user) == (today - datetime.timedelta(days=1)).isoformat()
    call = [{"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "get_weather", "arguments": {"location": "Tokyo", "unit": "celsius"}}}]}]
    out = Template("{{- range .Messages }}{{- range .ToolCalls }}{{ .Function.Arguments }}{{- end }}{{- end }}").execute(messages=call)
    assert js.loads(out) == {"location": "Tokyo", "unit": "celsius"}
    rng = "{{- range .Messages }}{{- range .ToolCalls }}{{- range $k, $v := .Function.Arguments }}{{ $k }}={{ $v }};{{- end }}{{- end }}{{- end }}"
    assert Template(rng).execute(messages=call) == "location=Tokyo;unit=celsius;"
    props = {"zeta": {"type": "string", "description": "zz", "enum": ["a", "b"]}, "alpha": {"type": ["number", "null"]},
             "obj": {"type": "object", "properties": {"k": {"type": "integer"}}}, "u": {"anyOf": [{"type": "string"}, {"type": "array", "items": {"type": "string"}}]}, "n": {}}
    tools = [{"type": "function", "function": {"name": "f", "description": "d", "parameters": {"type": "object", "required": ["zeta"], "properties": props}}}]
    head = "{{- range .Messages }}{{- end }}"
    assert js.loads(Template(head + "{{- range .Tools }}{{ .Function.Parameters.Properties }}{{ end }}").execute(messages=user, tools=tools)) == props
    assert js.loads(Template(head + "{{ range .Tools }}{{ json .Function.Parameters }}{{ end }}").execute(messages=user, tools=tools)) == tools[0]["function"]["parameters"]
    assert js.loads(Template(head + "{{ .Tools }}").execute(messages=user, tools=tools)) == tools
    each = head + "{{- range .Tools }}{{- range $name, $prop := .Function.Parameters.Properties }}{{ $name }}:{{ $prop.Type }}:{{ $prop.ToTypeScriptType }};{{- end }}{{- end }}"
    assert Template(each).execute(messages=user, tools=tools) == \
        "alpha:[number null]:number | null;n::any;obj:object:Record<string, any>;u::string | any[];zeta:string:string;"
    # consecutive messages of one role merge, tool answers never do (template_test.go:521-615)
    assert collate([{"role": "user", "content": "Hello"}, {"role": "user", "content": "How are you?"}]) == ("", [{"role": "user", "content": "Hello\n\nHow are you?"}])
    two = [{"role": "tool", "content": "sunny", "tool_name": "get_weather"}, {"role": "tool", "content": "72F", "tool_name": "get_temperature"}]
    assert collate(two) == ("", two)
    assert collate([{"role": "system", "content": "You are helpful"}] + user + two)[0] == "You are helpful"


def test_jinja_chat_template():
    t = JinjaChatTemplate("{{ bos_token }}{% for m in messages %}<{{ m.role }}>{{ m.content }}{% endfor %}"
                          "{% if add_generation_prompt %}<assistant>{% if enable_thinking %}<think>{% endif %}{% endif %}", bos_token="<s>")
    assert t.render([{"role": "user", "content": "hi"}], enable_thinking=True) == "<s><user>hi<assistant><think>"
    with pytest.raises(TemplateError):
        JinjaChatTemplate("{{ raise_exception('no') }}").render([])


def test_thinking_parser_streaming():
    p = ThinkingParser()
    chunks = ["  <th", "ink>  a", "bc </th", "ink>\n\n he", "llo"]
    got = [p.add(c) for c in chunks]
    assert "".join(t for t, _ in got) == "abc " and "".join(c for _, c in got) == "hello"
    p = ThinkingParser()
    assert p.add("no tags here") == ("", "no tags here")
    p = ThinkingParser(started=True)                       # the prompt already opened the block
    assert p.add("reason</think>answer") == ("reason", "answer")
    assert infer_tags("{{ if .Thinking }}<think>{{ .Thinking }}</think>{{ end }}{{ .Content }}") == ("<think>", "</think>")
    assert strip_thinking("<think>x</think>\n\nfinal") == "final"


def test_thinking_splitter_step_tables():
    """Streaming cases of the reference's splitter test (thinking/parser_test.go), as (input, thinking, content) steps."""
    cases = {
        "no tag": [("  abc", "", "  abc"), ("def", "", "def")],
        "content first nerfs the tag": [("  abc <think>def</think> ghi", "", "  abc <think>def</think> ghi")],
        "tag built up in pieces": [("  <th", "", ""), ("in", "", ""), ("k>a", "a", "")],
        "partial closing tag": [("<think>abc</th", "abc", ""), ("ink>def", "", "def")],
        "closing tag fake-out": [("<think>abc</th", "abc", ""), ("ing>def", "</thing>def", ""), ("ghi</thi", "ghi", ""), ("nk>jkl", "", "jkl")],
        "space after the block": [("  <think>abc</think>\n\ndef", "abc", "def")],
        "space after the block, later": [("  <think>abc</think>", "abc", ""), ("\n\ndef", "", "def")],
        "space is kept inside content": [("  <think>abc</think>\n\ndef ", "abc", "def "), (" ghi", "", " ghi")],
        "token by token": [("<think>", "", ""), ("\n", "", ""), ("</think>", "", ""), ("\n\n", "", ""), ("Hi", "", "Hi"), (" there", "", " there")],
        "leading space of the block": [("  <think>   \t ", "", ""), ("  these are some ", "these are some ", ""), ("thoughts </think>  ", "thoughts ", ""),
                                       ("  more content", "", "more content")],
        "one block only": [("<think>a</think><think>b</think>c", "a", "<think>b</think>c")],
        "space inside is kept at the end": [("<think> internal </think> world", "internal ", "world")],
    }
    for name, steps in cases.items():
        p = ThinkingParser()
        for i, (text, think, content) in enumerate(steps):
            assert p.add(text) == (think, content), (name, i)


def test_tool_parser():
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"properties": {"city": {}}}}}]
    p = ToolParser(tools, "<tool_call>")
    out = [p.add(c) for c in ["Sure <tool", '_call>{"name":"get_weather",', '"arguments":{"city":"Paris"}}</tool_call>']]
    calls = [c for cs, _ in out for c in cs]
    assert "".join(t for _, t in out).strip() == "Sure" and calls[0]["function"] == {"index": 0, "name": "get_weather", "arguments": {"city": "Paris"}}
    p = ToolParser(tools, "{")
    calls, text = p.add('{"name": "get_weather", "parameters": {"city": "Oslo"}}')
    assert calls and calls[0]["function"]["arguments"] == {"city": "Oslo"} and text == ""
    p = ToolParser(tools, "{")
    calls, text = p.add('The set {1, 2} is small')
    assert not calls and text == "The set {1, 2} is small"
    p = ToolParser(tools, "<tool_call>")
    calls, text = p.add('<tool_call>{"name": "unknown_tool", "arguments": {}}')
    assert not calls and "unknown_tool" in text
    assert infer_tag("{{ range .ToolCalls }}x{{ end }}") in ("{", "x")
    assert infer_tag('{{ if .ToolCalls }}<tool_call>\n{{ range .ToolCalls }}{"name"...{{ end }}{{ end }}') == "<tool_call>"


def test_harmony_parser_and_renderer():
    h = harmony.HarmonyParser()
    parts = ["<|channel|>analysis<|message|>think", "ing<|end|><|start|>assistant<|channel|>commentary to=functions.get_w ",
             '<|constrain|>json<|message|>{"a":1}<|call|>', "<|start|>assistant<|channel|>final<|mess", "age|>Hi!<|return|>"]
    th, ct, calls = "", "", []
    for p in parts:
        a, b, c = h.add(p)
        th, ct, calls = th + a, ct + b, calls + c
    assert th == "thinking" and ct == "Hi!" and calls[0]["function"]["name"] == "get_w" and calls[0]["function"]["arguments"] == {"a": 1}
    names = harmony.FunctionNameMap()
    assert names.convert("get-weather now") == "get_weather_now" and names.original("get_weather_now") == "get-weather now"
    assert names.convert("get_weather_now") == "get_weather_now_2"
    tools = [{"type": "function", "function": {"name": "get-w", "description": "d", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "n": {"type": "integer"}}, "required": ["city"]}}}]
    p = harmony.render_prompt([{"role": "system", "content": "be nice"}, {"role": "user", "content": "hi"},
                               {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "get-w", "arguments": {"city": "x"}}}]},
                               {"role": "tool", "tool_name": "get-w", "content": "sunny"}], tools, "high", today="2025-01-01")
    assert p.endswith("<|start|>assistant") and "Reasoning: high" in p and "type get_w = (_: {" in p and "city: string," in p and "n?: number," in p
    assert "<|start|>developer<|message|># Instructions\n\nbe nice" in p and 'to=functions.get_w <|constrain|>json<|message|>{"city":"x"}<|call|>' in p
    assert "<|start|>functions.get_w to=assistant<|channel|>commentary<|message|>sunny<|end|>" in p


def _bpe():
    b2u = _byte_to_unicode()
    tokens = [b2u[i] for i in range(256)] + ["he", "ll", "hell", "hello", "Ġw", "Ġwo", "Ġwor", "Ġworld", "<|eot|>", "<|eot|>x"]
    types = [1] * (len(tokens) - 2) + [3, 4]
    merges = ["h e", "l l", "he ll", "hell o", "Ġ w", "Ġw o", "Ġwo r", "Ġwor l", "Ġworl d"]
    tokens.insert(-2, "Ġworl")
    types.insert(-2, 1)
    return BPETokenizer(tokens, types, merges, "llama-bpe", bos=-1, eos=len(tokens) - 2)


def test_bpe_tokenizer():
    tk = _bpe()
    ids = tk.encode("hello world")
    assert [tk.tokens[i] for i in ids] == ["hello", "Ġworld"] and tk.decode(ids) == "hello world"
    ids = tk.encode("hello<|eot|>x!")                       # the longer special token wins
    assert tk.tokens[ids[1]] == "<|eot|>x" and tk.decode(ids) == "hello<|eot|>x!"
    assert tk.tokens[tk.encode("a<|eot|>", parse_special=True)[1]] == "<|eot|>"
    assert len(tk.encode("<|eot|>", parse_special=False)) > 1
    assert tk.decode(tk.encode("héllo ☃ 123456")) == "héllo ☃ 123456"
    assert tk.is_eog(tk.vocab["<|eot|>"])


def test_spm_tokenizer_and_gguf_selection():
    tokens = ["<unk>", "<s>", "</s>"] + [f"<0x{i:02X}>" for i in range(256)] + ["▁", "h", "e", "l", "o", "▁h", "he", "ll", "▁he", "llo", "▁hello", "w"]
    types = [2, 3, 3] + [6] * 256 + [1] * 12
    scores = [0.0] * 259 + [-1, -2, -2, -2, -2, -3, -4, -5, -6, -7, -0.5, -2]
    kv = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.token_type": types, "tokenizer.ggml.scores": scores,
          "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0}
    tk = tokenizer_from_gguf(kv)
    assert isinstance(tk, SPMTokenizer)
    ids = tk.encode("hello")
    assert ids[0] == 1 and tk.tokens[ids[1]] == "▁hello" and tk.decode(ids[1:]) == " hello"
    ids = tk.encode("hé", add_special=False)                # byte fallback for the unknown code point
    assert tk.decode(ids) == " hé" and any(tk.types[i] == 6 for i in ids)


def test_grammar_engine():
    m = GrammarMatcher(parse_gbnf(JSON_GRAMMAR))
    assert m.accepts('{"a": [1, 2.5e3, true, null, "x\\n"]}') and not m.accepts('{"a": }') and not m.accepts("[1]")
    g = parse_gbnf('root ::= "ab" [0-9]{2,3} ("x" | "y")? # tail\n')
    m = GrammarMatcher(g)
    assert m.accepts("ab12") and m.accepts("ab123y") and not m.accepts("ab1x") and not m.accepts("ab1234")
    with pytest.raises(GrammarError):
        parse_gbnf("root ::= missing")
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                               "tags": {"type": "array", "items": {"type": "string"}}, "k": {"enum": ["a", "b"]}},
              "required": ["name", "age"]}
    m = GrammarMatcher(parse_gbnf(json_schema_to_gbnf(schema)))
    assert m.accepts('{"name": "bob", "age": 3}') and m.accepts('{"name":"bob","age":3,"tags":["x","y"],"k":"a"}')
    assert not m.accepts('{"age": 3}') and not m.accepts('{"name":"b","age":"3"}')
    m.advance('{"name":"bob","age":3}')
    assert m.can_end()
    assert grammar_for_format(None) is None and grammar_for_format("json") == JSON_GRAMMAR and "root" in grammar_for_format({"type": "object"})
    with pytest.raises(GrammarError):
        grammar_for_format("yaml")
    tk = _bpe()
    gr = Grammar('root ::= "hello" " world"?', tk)
    assert gr.allows(tk.vocab["hello"]) and not gr.allows(tk.vocab["Ġworld"])
    gr.accept(tk.vocab["hello"])
    assert gr.allows(tk.vocab["Ġworld"]) and gr.allows(tk.eos) and not gr.done()
    gr.accept(tk.vocab["Ġworld"])
    assert gr.done()


def _trained_bpe(corpus: str, n_merges: int) -> BPETokenizer:
    """A small byte-level BPE table learnt from ``corpus`` (most frequent pair first), so that merges chain as in real vocabularies."""
    import collections

    import regex
    b2u = _byte_to_unicode()
    tokens = [b2u[i] for i in range(256)]
    words = collections.Counter(tuple(b2u[b] for b in w.encode("utf-8")) for w in regex.findall(r" ?[^\s]+|\s+", corpus))
    merges = []
    for _ in range(n_merges):
        pairs = collections.Counter()
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += c
        if not pairs:
            break
        (a, b), _ = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        merges.append(f"{a} {b}")
        tokens.append(a + b)
        nw = collections.Counter()
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            nw[tuple(out)] += c
        words = nw
    return BPETokenizer(tokens, [1] * len(tokens), merges, "llama-bpe")


def test_native_bpe_merge_loop_matches_python():
    from ollama_b200.utils import hostlib
    if hostlib.lib() is None:
        pytest.skip("host library not built")
    corpus = ("the quick brown fox jumps over the lazy dog. " * 3 + "aaaa aaa aaaaa banana bandana ananas. "
              "Tokenisation of naïve café text — with ☃ snowmen, 12345 67890 numbers and CamelCaseIdentifiers_like_this(). ") * 4
    tk = _trained_bpe(corpus, 300)
    assert tk._native_table() is not None
    text = corpus + " unseen wörds zzzz aaaaaaaaaaaaaaaa " + "x" * 300 + " done"
    native = tk.encode(text, add_special=False)
    tk2 = _trained_bpe(corpus, 300)
    tk2._native = False                                  # forces the Python merge loop
    assert native == tk2.encode(text, add_special=False) and tk.decode(native) == text
    assert len(native) < len(text.encode()) // 2          # merges really happened


_TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "Weather for a city", "parameters": {
    "type": "object", "required": ["city"], "properties": {
        "city": {"type": "string", "description": "City name"}, "days": {"type": "integer"}, "metric": {"type": "boolean"},
        "tags": {"type": "array"}, "opts": {"type": ["object", "null"]}, "ratio": {"type": "number"}}}}}]


def _feed(parser, text, step):
    """Stream ``text`` in pieces of ``step`` characters; returns (content, thinking, calls)."""
    c, t, calls = "", "", []
    for i in range(0, len(text), step):
        a, b, k = parser.add(text[i:i + step], i + step >= len(text))
        c, t, calls = c + a, t + b, calls + k
    return c, t, calls


@pytest.mark.parametrize("step", [1, 3, 7, 1000])
def test_builtin_parsers_split_streams_the_same_way_at_every_chunking(step):
    from ollama_b200.text.builtin import parser_for, typed_value
    out = ("I will look it up.\n\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n3\n</parameter>\n"
           "<parameter=metric>\nTrue\n</parameter>\n<parameter=tags>\n[\"a\", 1]\n</parameter>\n<parameter=opts>\nnull\n</parameter>\n"
           "<parameter=ratio>\n2.0\n</parameter>\n<parameter=note>\nline 1\nline 2\n</parameter>\n</function>\n</tool_call>")
    c, t, calls = _feed(parser_for("qwen3-coder", _TOOLS), out, step)
    assert c == "I will look it up." and t == "" and len(calls) == 1
    assert calls[0]["function"] == {"name": "get_weather", "arguments": {"city": "Paris", "days": 3, "metric": True, "tags": ["a", 1], "opts": None,
                                                                         "ratio": 2, "note": "line 1\nline 2"}}
    # a reasoning model: the prompt ended inside <think>, some checkpoints repeat the tag
    for lead in ("", "<think>"):
        out = lead + "Let me think.\nOK.</think>\n\nThe answer is 4 < 5.\n<tool_call>\n{\"name\": \"get_weather\", \"arguments\": {\"city\": \"Oslo\"}}\n</tool_call>"
        c, t, calls = _feed(parser_for("qwen3-thinking", _TOOLS, None), out, step)
        assert t == "Let me think.\nOK." and c == "The answer is 4 < 5." and calls[0]["function"] == {"name": "get_weather", "arguments": {"city": "Oslo"}}
    # thinking switched off, or an assistant prefill: everything is content; without tools the call markup stays text
    c, t, calls = _feed(parser_for("qwen3-thinking", None, False), "plain <b>text</b> <tool_call>x</tool_call>", step)
    assert (c, t, calls) == ("plain <b>text</b> <tool_call>x</tool_call>", "", [])
    assert _feed(parser_for("qwen3-thinking", None, None, prefill="So"), " it goes", step)[0] == " it goes"
    out = "[THINK]hmm[/THINK]Sure.[TOOL_CALLS]get_weather[ARGS]{\"city\": \"Rome {x}\", \"n\": {\"a\": \"}\"}}[TOOL_CALLS]get_weather[ARGS]{\"city\": \"Bern\"}"
    c, t, calls = _feed(parser_for("ministral", _TOOLS), out, step)
    assert (c, t) == ("Sure.", "hmm") and [k["function"]["arguments"]["city"] for k in calls] == ["Rome {x}", "Bern"]
    # malformed or unterminated calls come back as the text that was produced
    c, _, calls = _feed(parser_for("qwen3", _TOOLS), "a <tool_call>not json</tool_call> b <tool_call>{\"name\"", step)
    assert calls == [] and c == "a<tool_call>not json</tool_call>b<tool_call>{\"name\""
    assert _feed(parser_for("passthrough"), " raw <think> ", step) == (" raw <think> ", "", [])
    assert parser_for("unknown-family") is None and parser_for(None) is None
    assert typed_value("12", ["string", "integer"]) == 12 and typed_value("x", ["integer"]) == "x" and typed_value("maybe", ["boolean"]) is False
    assert typed_value("1.5", ["number"]) == 1.5 and typed_value("{\"a\":1}", ["object"]) == {"a": 1} and typed_value("NULL", ["string"]) is None


def test_qwen3_coder_renderer():
    from ollama_b200.text.builtin import render_qwen3_coder, renderer_for
    assert callable(renderer_for("qwen3-coder")) and renderer_for("nope") is None
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "system", "content": "ignored"}, {"role": "user", "content": "Weather?"},
            {"role": "assistant", "content": "Checking.", "tool_calls": [{"function": {"name": "get_weather", "arguments": {"city": "Paris", "days": 2, "opts": {"a": 1}}}}]},
            {"role": "tool", "content": "sunny"}, {"role": "tool", "content": "22C"}]
    p = render_qwen3_coder(msgs, _TOOLS)
    assert p.startswith("<|im_start|>system\nBe brief.\n\n# Tools\n\nYou have access to the following functions:\n\n<tools>\n<function>\n<name>get_weather</name>\n"
                        "<description>Weather for a city</description>\n<parameters>\n<parameter>\n<name>city</name>\n<type>string</type>\n<description>City name</description>\n</parameter>")
    assert "<type>[\"object\",\"null\"]</type>" in p and "\n<required>[\"city\"]</required>\n</parameters>\n</function>\n</tools>" in p and "ignored" not in p
    assert ("<|im_start|>assistant\nChecking.\n\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n2\n</parameter>\n"
            "<parameter=opts>\n{\"a\":1}\n</parameter>\n</function>\n</tool_call><|im_end|>\n") in p
    assert p.endswith("<|im_start|>user\n<tool_response>\nsunny\n</tool_response>\n<tool_response>\n22C\n</tool_response><|im_end|>\n<|im_start|>assistant\n")
    # no system message, no tools: plain ChatML; a trailing assistant message stays open
    assert render_qwen3_coder([{"role": "user", "content": "hi"}]) == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert render_qwen3_coder([{"role": "user", "content": "hi"}, {"role": "assistant", "content": "He"}]).endswith("<|im_start|>assistant\nHe")
    assert "You are Qwen, a helpful AI assistant" in render_qwen3_coder([{"role": "user", "content": "hi"}], _TOOLS)


def _reference_template_dir():
    """The reference's template directory, when OLLAMA_REFERENCE_DIR names a checkout of the reference (golden prompt files)."""
    import os
    d = os.path.join(os.environ.get("OLLAMA_REFERENCE_DIR", ""), "template")
    return d if os.path.isdir(os.path.join(d, "testdata")) else None


@pytest.mark.skipif(_reference_template_dir() is None, reason="OLLAMA_REFERENCE_DIR does not name a checkout of the reference")
def test_go_templates_reproduce_the_reference_golden_prompts():
    """Every bundled chat layout of the reference (template/*.gotmpl) rendered for its three golden conversations
    (template/template_test.go:66-140) gives the bytes stored under template/testdata/<layout>/<case>."""
    import glob
    import os
    ref = _reference_template_dir()
    convs = {
        "user": [("user", "Hello, how are you?")],
        "user-assistant-user": [("user", "Hello, how are you?"), ("assistant", "I'm doing great. How can I help you today?"),
                                ("user", "I'd like to show off how chat templating works!")],
        "system-user-assistant-user": [("system", "You are a helpful assistant."), ("user", "Hello, how are you?"),
                                       ("assistant", "I'm doing great. How can I help you today?"),
                                       ("user", "I'd like to show off how chat templating works!")],
    }
    files = sorted(glob.glob(os.path.join(ref, "*.gotmpl")))
    assert len(files) >= 15
    checked = 0
    for f in files:
        name = os.path.basename(f)
        with open(f, encoding="utf-8") as fh:
            t = Template(fh.read())
        for case, conv in convs.items():
            golden = os.path.join(ref, "testdata", name, case)
            if not os.path.exists(golden):
                continue
            with open(golden, encoding="utf-8") as fh:
                want = fh.read()
            got = t.execute(messages=[{"role": r, "content": c} for r, c in conv])
            assert got == want, (name, case)
            checked += 1
    assert checked >= 45


def _reference_llama_vocab():
    import os
    d = os.path.join(os.environ.get("OLLAMA_REFERENCE_DIR", ""), "tokenizer", "testdata")
    return d if os.path.exists(os.path.join(d, "llama3.2", "encoder.json")) else None


@pytest.mark.skipif(_reference_llama_vocab() is None, reason="OLLAMA_REFERENCE_DIR does not name a checkout of the reference")
def test_bpe_on_the_llama3_vocabulary_matches_the_reference_ids():
    """The reference's tokenizer fixture (a full Llama-3 vocabulary with 280 k merges) and the ids its tests expect
    (tokenizer/bytepairencoding_test.go:82-215): digit grouping, special tokens, and on a long text the C++ merge loop
    against the Python one."""
    import json as _json
    import os
    d = _reference_llama_vocab()
    with open(os.path.join(d, "llama3.2", "encoder.json"), encoding="utf-8") as f:
        vocab = _json.load(f)
    tokens = [""] * len(vocab)
    for t, i in vocab.items():
        tokens[i] = t
    types = [1] * len(tokens)
    for t in ("<|begin_of_text|>", "<|end_of_text|>"):
        if t not in vocab:
            vocab[t] = len(tokens)
            tokens.append(t)
            types.append(3)
    with open(os.path.join(d, "llama3.2", "vocab.bpe"), encoding="utf-8") as f:
        merges = [l.rstrip("\n") for l in f if not l.startswith("#") and l.strip()]

    def make():
        return BPETokenizer(tokens, types, merges, "llama-bpe", bos=vocab["<|begin_of_text|>"], eos=vocab["<|end_of_text|>"])

    tk = make()
    enc = lambda s: tk.encode(s, add_special=False)      # noqa: E731
    assert enc("hello world") == [15339, 1917]
    for n, want in ((1, [15]), (2, [410]), (3, [931]), (4, [931, 15]), (5, [931, 410]), (7, [931, 931, 15]), (12, [931] * 4), (17, [931] * 5 + [410])):
        assert enc("0" * n) == want, n
    assert enc("<|begin_of_text|>A B!") == [128000, 32, 426, 0]
    assert enc("<|begin_of_text|>A<|end_of_text|>B<|begin_of_text|>!<|end_of_text|>") == [128000, 32, 128001, 33, 128000, 0, 128001]
    with open(os.path.join(d, "war-and-peace.txt"), encoding="utf-8") as f:
        text = f.read()[:200_000]
    assert tk._native_table() is not None
    native = enc(text)
    slow = make()
    slow._native = False
    assert native == slow.encode(text, add_special=False) and tk.decode(native) == text
    assert len(native) < len(text) / 3


@pytest.mark.skipif(_reference_template_dir() is None, reason="OLLAMA_REFERENCE_DIR does not name a checkout of the reference")
def test_jinja_engine_runs_the_known_chat_templates():
    """The Jinja chat templates the reference recognises (template/index.json, 37 real-world layouts): every one parses
    and renders three conversations; the only failures allowed are the templates' own ``raise_exception`` calls, and the
    rendering contains every message of the conversation."""
    import json as _json
    import os
    from ollama_b200.text.template import JinjaChatTemplate
    with open(os.path.join(_reference_template_dir(), "index.json"), encoding="utf-8") as f:
        idx = _json.load(f)
    assert len(idx) >= 30
    convs = [[("user", "Hello, how are you?")],
             [("user", "Hello, how are you?"), ("assistant", "I'm doing great."), ("user", "Show me templating!")],
             [("system", "You are a helpful assistant."), ("user", "Hello, how are you?"), ("assistant", "I'm doing great."), ("user", "Show me templating!")]]
    rendered = refused = 0
    for e in idx:
        t = JinjaChatTemplate(e["template"], e.get("bos_token", "<s>"), e.get("eos_token", "</s>"))
        for conv in convs:
            try:
                out = t.render([{"role": r, "content": c} for r, c in conv], None, True)
            except TemplateError as ex:
                assert any(w in str(ex).lower() for w in ("system", "alternate", "role")), (e["name"], ex)
                refused += 1
                continue
            rendered += 1
            for r, c in conv:
                if r != "system":
                    assert c in out, (e["name"], c)
    assert rendered >= 100 and refused <= 8


def test_builtin_parsers_are_chunking_invariant_under_random_splits():
    """Property: however the output is cut into chunks, the concatenated (content, thinking, calls) is the same."""
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import strategies as stg
    from ollama_b200.text.builtin import parser_for
    outputs = {
        "qwen3-coder": "Sure <b>.\n\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n</function>\n</tool_call>\n\nand <tool_ca not a call",
        "qwen3-thinking": "<think>\nstep 1 < step 2\n</think>\n\nAnswer: 4.\n<tool_call>\n{\"name\": \"get_weather\", \"arguments\": {\"city\": \"Oslo\"}}\n</tool_call>\n",
        "qwen3": "plain </think> text <tool_call>{\"name\": \"get_weather\", \"arguments\": {\"days\": 2}}</tool_call> tail  ",
        "ministral": "[THINK]a [b] c[/THINK] ok [TOOL_CALLS]get_weather[ARGS]{\"city\": \"R}\"} rest",
    }
    whole = {n: parser_for(n, _TOOLS).add(t, True) for n, t in outputs.items()}

    @hyp.settings(max_examples=150, deadline=None)
    @hyp.given(stg.sampled_from(sorted(outputs)), stg.lists(stg.integers(min_value=1, max_value=40), min_size=1, max_size=60))
    def check(name, sizes):
        text, p = outputs[name], parser_for(name, _TOOLS)
        c, t, calls, i, k = "", "", [], 0, 0
        while i < len(text):
            n = sizes[k % len(sizes)]
            k += 1
            a, b, cc = p.add(text[i:i + n], i + n >= len(text))
            c, t, calls, i = c + a, t + b, calls + cc, i + n
        assert (c, t, calls) == whole[name]

    check()
    assert whole["qwen3-coder"][2][0]["function"]["arguments"] == {"city": "Paris"} and whole["ministral"][1] == "a [b] c"


def test_parsers_reject_mutated_input_with_their_own_error_types():
    """Mutations of valid Go templates, GBNF grammars and Modelfiles either still work or fail with the error type the
    server turns into a 400 (TemplateError, GrammarError, ModelfileError / OptionError): no other exception escapes."""
    import random
    from ollama_b200.api.types import OptionError
    from ollama_b200.store.modelfile import ModelfileError, parse_modelfile
    rnd = random.Random(1)

    def mutate(s):
        b = list(s)
        for _ in range(rnd.randint(1, 3)):
            op, i = rnd.random(), rnd.randrange(len(b)) if b else 0
            if op < 0.4 and b:
                b[i] = rnd.choice('{}|.()"$ -:=\\n' + s[rnd.randrange(len(s))])
            elif op < 0.7 and b:
                del b[i:i + rnd.randint(1, 5)]
            else:
                b.insert(i, rnd.choice(["{{", "}}", "{{-", " end ", '"', "(", ")", "|", "range ", "if ", "::=", "[", "\\\\"]))
        return "".join(b)

    tmpls = ['{{- $system := "" }}{{- range .Messages }}{{- if eq .Role "system" }}{{ $system = .Content }}{{- else if eq .Role "user" }}'
             '[INST] {{ if $system }}{{ $system }}\\n\\n{{ end }}{{ .Content }}[/INST]{{- else }} {{ .Content }}</s>{{- end }}{{- end }}',
             '{{ if .System }}<|im_start|>system\\n{{ .System }}<|im_end|>\\n{{ end }}{{ range $i, $m := .Messages }}{{ if gt $i 0 }}\\n{{ end }}'
             '<|im_start|>{{ $m.Role }}\\n{{ $m.Content }}{{ if lt (len (slice $.Messages $i)) 2 }}<|im_end|>{{ end }}{{ end }}']
    msgs = [{"role": "system", "content": "s"}, {"role": "user", "content": "u"}, {"role": "assistant", "content": "a"}, {"role": "user", "content": "q"}]
    worked = 0
    for _ in range(600):
        src = mutate(rnd.choice(tmpls))
        try:
            Template(src).execute(messages=[dict(m) for m in msgs])
            worked += 1
        except TemplateError:
            pass
    assert 0 < worked < 600
    for _ in range(400):
        try:
            GrammarMatcher(parse_gbnf(mutate(JSON_GRAMMAR))).accepts('{"a": [1, true]}')
        except GrammarError:
            pass
    mf = 'FROM llama3\\nTEMPLATE """{{ .Prompt }}"""\\nSYSTEM "hi"\\nPARAMETER temperature 0.5\\nPARAMETER stop "x"\\nMESSAGE user hello\\nADAPTER ./a.gguf\\n'
    for _ in range(400):
        try:
            parse_modelfile(mutate(mf)).create_request()
        except (ModelfileError, OptionError):
            pass


def test_functiongemma_renderer_and_parser():
    """Expected prompts are the golden strings of the reference's renderer tests (model/renderers/functiongemma_test.go)."""
    from ollama_b200.text.builtin import parser_for, render_functiongemma
    weather = [{"type": "function", "function": {"name": "get_weather", "description": "Get weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string", "description": "City"}}}}}]
    decl = ("<start_function_declaration>declaration:get_weather{description:<escape>Get weather<escape>,parameters:{properties:{city:{description:"
            "<escape>City<escape>,type:<escape>STRING<escape>}},type:<escape>OBJECT<escape>}}<end_function_declaration>")
    hello = [{"role": "user", "content": "Hello!"}]
    assert render_functiongemma(hello) == "<bos><start_of_turn>user\nHello!<end_of_turn>\n<start_of_turn>model\n"
    assert render_functiongemma([{"role": "system", "content": "You are helpful"}] + hello) == \
        "<bos><start_of_turn>developer\nYou are helpful<end_of_turn>\n<start_of_turn>user\nHello!<end_of_turn>\n<start_of_turn>model\n"
    assert render_functiongemma([]) == "<bos><start_of_turn>model\n"
    q = [{"role": "user", "content": "Weather?"}]
    assert render_functiongemma([{"role": "system", "content": "You are a weather expert."}] + q, weather) == \
        ("<bos><start_of_turn>developer\nYou are a weather expert.\nYou can do function calling with the following functions:" + decl +
         "<end_of_turn>\n<start_of_turn>user\nWeather?<end_of_turn>\n<start_of_turn>model\n")
    head = "<bos><start_of_turn>developer\nYou can do function calling with the following functions:" + decl + "<end_of_turn>\n<start_of_turn>user\nWeather?<end_of_turn>\n<start_of_turn>model\n"
    assert render_functiongemma(q, weather) == head
    call = {"role": "assistant", "content": "Let me check.", "tool_calls": [{"function": {"name": "get_weather", "arguments": {"city": "Paris"}}}]}
    assert render_functiongemma(q + [call, {"role": "tool", "content": "Sunny"}], weather) == \
        head + "Let me check.<start_function_call>call:get_weather{city:<escape>Paris<escape>}<end_function_call><start_function_response>response:get_weather{<escape>Sunny<escape>}<end_function_response>"
    add = [{"type": "function", "function": {"name": "add", "description": "Add numbers", "parameters": {
        "type": "object", "properties": {"a": {"type": "number"}, "b": {"type": "number"}}}}}]
    got = render_functiongemma([{"role": "user", "content": "Add"}, {"role": "assistant", "tool_calls": [{"function": {"name": "add", "arguments": {"b": 2, "a": 1.0}}}]},
                                {"role": "tool", "content": "3"}], add)
    assert got.endswith("<start_of_turn>model\n<start_function_call>call:add{a:1,b:2}<end_function_call><start_function_response>response:add{<escape>3<escape>}<end_function_response>")
    assert "a:{description:<escape><escape>,type:<escape>NUMBER<escape>},b:{description:<escape><escape>,type:<escape>NUMBER<escape>}" in got
    req = [{"type": "function", "function": {"name": "get_weather", "description": "Gets the weather for a given city", "parameters": {
        "type": "object", "required": ["city"], "properties": {"city": {"type": "string", "description": "City Name"}, "country": {"type": "string", "description": "Country Name"}}}}}]
    assert ("country:{description:<escape>Country Name<escape>,type:<escape>STRING<escape>}},required:[<escape>city<escape>],type:<escape>OBJECT<escape>}}"
            "<end_function_declaration>") in render_functiongemma(q, req)
    # the parser reads what the renderer writes, nested values included, at any chunking
    out = ("I will call it.<start_function_call>call:plan{city:<escape>Paris, France<escape>,days:3,ratio:1.5,ok:true,tags:[<escape>a,b<escape>,2],"
           "opts:{unit:<escape>C<escape>,deep:{x:1}}}<end_function_call>")
    for step in (1, 5, 1000):
        c, t, calls = _feed(parser_for("functiongemma", weather), out, step)
        assert c == "I will call it." and t == "" and calls == [{"function": {"name": "plan", "arguments": {
            "city": "Paris, France", "days": 3, "ratio": 1.5, "ok": True, "tags": ["a,b", 2], "opts": {"unit": "C", "deep": {"x": 1}}}}}]


def test_harmony_header_forms():
    """Header variants of the reference's parser test (harmony/harmonyparser_test.go:9-92): recipient before or after the
    channel, a constrain tag with or without a space, extra tokens after the recipient."""
    cases = [("assistant<|channel|>analysis", "analysis", ""),
             ("assistant<|channel|>analysis to=functions.get_weather", "analysis", "functions.get_weather"),
             ("assistant to=functions.get_weather<|channel|>analysis", "analysis", "functions.get_weather"),
             ("to=functions.get_weather<|channel|>analysis", "analysis", "functions.get_weather"),
             ("assistant to=functions.get_weather abc<|channel|>analysis", "analysis", "functions.get_weather"),
             ("assistant<|channel|>commentary to=functions.get_weather <|constrain|>json", "commentary", "functions.get_weather"),
             ("assistant to=functions.get_weather<|channel|>commentary <|constrain|>json", "commentary", "functions.get_weather"),
             ("assistant<|channel|>commentary to=functions.get_weather<|constrain|>json", "commentary", "functions.get_weather"),
             ("assistant to=functions.get_weather<|channel|>commentary<|constrain|>json", "commentary", "functions.get_weather")]
    for header, channel, recipient in cases:
        p = harmony.HarmonyParser(harmony.FunctionNameMap())
        p._parse_header(header)
        assert (p.channel, p.recipient) == (channel, recipient), header
    # and end to end: a call in the commentary channel with a constrain tag glued to the recipient
    p = harmony.HarmonyParser(harmony.FunctionNameMap())
    th, ct, calls = "", "", []
    for piece in ("<|channel|>analysis<|message|>need weather<|end|><|start|>assistant<|channel|>commentary to=functions.get_weather<|constrain|>json<|message|>",
                  '{"city":"Paris"}<|call|>'):
        a, b, c = p.add(piece)
        th, ct, calls = th + a, ct + b, calls + c
    assert th == "need weather" and ct == "" and calls[0]["function"]["name"] == "get_weather" and calls[0]["function"]["arguments"] == {"city": "Paris"}


def test_harmony_function_name_map_follows_the_reference_table():
    """harmony/harmonyparser_test.go:473-560."""
    M = harmony.FunctionNameMap
    for name, want in (("get weather", "get_weather"), ("get-weather", "get_weather"), ("get.weather", "get_weather"), ("get weather!", "get_weather"),
                       ("a🫠bc", "abc"), ("🫠", "unnamed"), ("123", "_123"), ("$", "$"), ("𝓸𝓵𝓵𝓪𝓶𝓪", "𝓸𝓵𝓵𝓪𝓶𝓪"), ("ⓞⓛⓛⓐⓜⓐ123", "_123")):
        assert M.valid_chars(name) == want, name
    for names, want in ((["get weather", "get weather"], ["get_weather", "get_weather_2"]),
                        (["get weather", "get_weather", "get-weather", "something-different"], ["get_weather", "get_weather_2", "get_weather_3", "something_different"]),
                        (["a", "a", "b", "a", "a", "b", "a"], ["a", "a_2", "b", "a_3", "a_4", "b_2", "a_5"]),
                        (["browser.open", "python", "not.a.built-in.function", "browser.not_a_real_built_in"],
                         ["browser.open", "python", "not_a_built_in_function", "browser_not_a_real_built_in"])):
        m = M()
        got = [m.add(n) for n in names]
        assert got == want and all(m.original(h) == n for n, h in zip(names, got))
    m = M()
    assert m.convert("get-w") == "get_w" and m.convert("get-w") == "get_w" and m.original("get_w") == "get-w"      # lookups do not rename


def test_generic_tool_parser_on_the_reference_cases():
    """A selection of the reference's tool-parser table (tools/tools_test.go:156-790): tag and bare-JSON forms, lists,
    names that are prefixes of other names, arguments before the name, JSON that is not a call, split input."""
    def tool(n, props=()):
        return {"type": "function", "function": {"name": n, "description": "d", "parameters": {"type": "object", "properties": {k: {"type": "string"} for k in props}}}}
    tools = [tool("get_temperature", ("format", "city")), tool("get_conditions", ("location",)), tool("say_hello"), tool("say_hello_world"),
             tool("get_address", ("location",)), tool("add", ("a", "b"))]

    def run(tag, inputs):
        p, c, calls = ToolParser(tools, tag), "", []
        for s in inputs:
            k, t = p.add(s)
            calls, c = calls + k, c + t
        return c + p.flush(), [(x["function"]["name"], x["function"]["arguments"]) for x in calls]

    london = ("get_temperature", {"city": "London", "format": "fahrenheit"})
    tokyo = ("get_conditions", {"location": "Tokyo"})
    cases = [
        ("<tool_call>", ['<tool_call>{"name": "get_conditions", "arguments": {"location": "San Francisco"}}</tool_call>'], "", [("get_conditions", {"location": "San Francisco"})]),
        ("<tool_call>", ['Let me check the weather. <tool_call>{"name": "get_temperature", "arguments": {"city": "New York"}}</tool_call>'],
         "Let me check the weather. ", [("get_temperature", {"city": "New York"})]),
        ("<tool_call>", ["Let me say hello to the user. I'll use the say_hello tool. "], "Let me say hello to the user. I'll use the say_hello tool. ", []),
        ("[TOOL_CALLS]", ['[TOOL_CALLS] [{"name": "get_temperature", "arguments": {"city": "London", "format": "fahrenheit"}}, '
                          '{"name": "get_conditions", "arguments": {"location": "Tokyo"}}][/TOOL_CALLS]'], "", [london, tokyo]),
        ("<tool_call>", ['Okay, let\'s call both tools! <tool_call>{"name": "get_temperature", "arguments": {"city": "London", "format": "fahrenheit"}}</tool_call>'
                         '<tool_call>{"name": "get_conditions", "arguments": {"location": "Tokyo"}}</tool_call>'], "Okay, let's call both tools! ", [london, tokyo]),
        ("<tool_call>", ['<tool_call>{"name": "say_hello", "arguments": {}}</tool_call><tool_call>{"name": "get_temperature", "arguments": '
                         '{"city": "London", "format": "fahrenheit"}}</tool_call>'], "", [("say_hello", {}), london]),
        ("{", ['{"name": "get_temperature", "arguments": {"city": "London", "format": "fahrenheit"}}'], "", [london]),
        ("{", ['{"name": "search", ', '"arguments": {"query": "What is the capital of Canada?"}}'],
         '{"name": "search", "arguments": {"query": "What is the capital of Canada?"}}', []),
        ("<tool_call>", ['<tool_call>{"name": "say_hello_world", "arguments": {}}'], "", [("say_hello_world", {})]),
        ("<tool_call>", ['<tool_call>{"name": "say_hello', '_world", ', '"arguments": {}}</tool_call>'], "", [("say_hello_world", {})]),
        ("<tool_call>", ['<tool_call>{"arguments": {"a": "5", "b": "10"}, "name": "add"}</tool_call>'], "", [("add", {"a": "5", "b": "10"})]),
    ]
    for tag, inputs, content, calls in cases:
        assert run(tag, inputs) == (content, calls), inputs
