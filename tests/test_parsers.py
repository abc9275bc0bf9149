"""Built-in output parsers on the reference's own cases.

``tests/data/parser_cases.json`` restates tables of the reference's parser tests (model/parsers/*_test.go) as data:
``streams`` are completions (whole, or in the chunks the reference's test feeds) with the content, reasoning and calls
expected from them; ``glm_calls``, ``olmo3_calls`` and ``olmo3_values`` are the bodies of single tool calls.  A few rows
differ by design and are listed with the reason; every other row has to match, at the reference's chunking and at
three others.
"""
import json
import os

import pytest

from ollama_b200.text import builtin as B

with open(os.path.join(os.path.dirname(__file__), "data", "parser_cases.json"), encoding="utf-8") as _f:
    DATA = json.load(_f)

# This parser gives the same answer however the stream is cut into chunks, and releases held text when the stream ends.
BY_DESIGN = {
    ("cogito_test.go", "split_tool_calls_begin_tag_conservative_parsing"): "a mark split across two chunks is still a mark",
    ("deepseek3_test.go", "streaming_with_split_tags"): "white space around a call block does not depend on where the chunks end",
    ("deepseek3_test.go", "partial_think_tag_at_end_with_thinking"): "a held piece of a mark is released when the stream ends",
    ("deepseek3_test.go", "consecutive_tool_calls"): "a second block of calls is parsed like the first",
    ("qwen3vl_nonthinking_test.go", "partial thinking incomplete"): "a held piece of a mark is released when the stream ends",
    ("qwen3vl_thinking_test.go", "partial thinking incomplete"): "a held piece of a mark is released when the stream ends",
}
TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {}}}}]


def _num(v):
    if isinstance(v, float) and v == int(v):
        return int(v)
    if isinstance(v, dict):
        return {k: _num(x) for k, x in v.items()}
    return [_num(x) for x in v] if isinstance(v, list) else v


def _same(a, b):
    return json.dumps(_num(a), sort_keys=True) == json.dumps(_num(b), sort_keys=True)


def _run(case, chunks):
    p = B.parser_for(case["parser"], case.get("tools") or TOOLS if case["parser"] != "cogito" else case.get("tools"), case.get("think"), case.get("prefill", ""), case.get("after_tool", False))
    content = thinking = ""
    calls = []
    for i, ch in enumerate(chunks):
        c, t, k = p.add(ch, i == len(chunks) - 1)
        content, thinking, calls = content + c, thinking + t, calls + k
    return content, thinking, [{"name": k["function"]["name"], "arguments": k["function"]["arguments"]} for k in calls]


def _cut(text, n):
    return [text[i:i + n] for i in range(0, len(text), n)] or [""]


@pytest.mark.parametrize("name", sorted({c["parser"] for c in DATA["streams"]}))
def test_parser_streams_match_the_reference_cases(name):
    rows = [c for c in DATA["streams"] if c["parser"] == name and (c["source"], c["case"]) not in BY_DESIGN]
    assert rows
    for c in rows:
        whole = "".join(c["chunks"])
        for chunks in (c["chunks"], [whole], _cut(whole, 1), _cut(whole, 5)):
            content, thinking, calls = _run(c, chunks)
            if c.get("loose"):                          # the reference's event tables stop before the stream ends: trailing space is still held there
                content, thinking, want = content.strip(), thinking.strip(), (c["content"].strip(), c["thinking"].strip())
            else:
                want = (c["content"], c["thinking"])
            assert (content, thinking) == want, (c["source"], c["case"], chunks)
            assert _same(calls, c["calls"]), (c["source"], c["case"])


def test_rows_that_differ_by_design_really_differ():
    for c in DATA["streams"]:
        if (c["source"], c["case"]) in BY_DESIGN:
            content, thinking, calls = _run(c, c["chunks"])
            assert (content, thinking) != (c["content"], c["thinking"]) or not _same(calls, c["calls"]), c["case"]


def test_single_call_bodies():
    for c in DATA["glm_calls"]:
        got = B._glm_call(c["tools"])(c["body"])
        assert got is not None and got["function"]["name"] == c["name"] and _same(got["function"]["arguments"], c["arguments"]), c["case"]
    for c in DATA["olmo3_calls"]:
        got = B._pythonic_calls(c["body"]) or []
        assert _same([{"name": k["function"]["name"], "arguments": k["function"]["arguments"]} for k in got], c["calls"]), c["case"]
    for c in DATA["olmo3_values"]:
        got = B._pythonic_calls("f(x=" + c["text"] + ")")
        assert got is not None and _same(got[0]["function"]["arguments"]["x"], c["value"]), c["case"]
    for c in DATA["lfm2_calls"]:
        got = B._python_call_list(c["body"])
        if c["error"]:
            assert not got, c["case"]
        else:
            assert _same([{"name": k["function"]["name"], "arguments": k["function"]["arguments"]} for k in got or []], c["calls"]), c["case"]
    assert B._pythonic_calls('book(from="SFO", class="eco", to=None)')[0]["function"]["arguments"] == {"from": "SFO", "class": "eco", "to": None}
    assert B._pythonic_calls("not a call") is None and B._pythonic_calls("f(1, 2)") is None
    assert B._cogito_call("function<｜tool▁sep｜>w\n```json\n{\"a\": 1}\n```")["function"] == {"name": "w", "arguments": {"a": 1}}
    assert B._cogito_call("function<｜tool▁sep｜>w {}") is None and B._deepseek_call("w<｜tool▁sep｜>[1]") is None


def test_registry_and_initial_state():
    for name in B.PARSERS:
        assert B.parser_for(name, TOOLS) is not None
    # reasoning: cogito only on request and never with tools; glm-4.7 unless switched off; a continued answer is never reasoning
    assert B.parser_for("cogito", None, True).state == "thinking" and B.parser_for("cogito", TOOLS, True).state == "content"
    assert B.parser_for("cogito", None, None).state == "content" and B.parser_for("deepseek3", TOOLS, True).state == "thinking"
    assert B.parser_for("glm-4.7", None, None).state == "thinking" and B.parser_for("glm-4.7", None, False).state == "content"
    assert B.parser_for("glm-4.6", None, None).state == "content"
    assert B.parser_for("olmo3-think", None, None, prefill="So").state == "content" and B.parser_for("qwen3-vl-thinking", None, False).state == "thinking"
    # a call inside the reasoning block of qwen3-vl ends the block
    c, t, k = B.parser_for("qwen3-vl-thinking", TOOLS).add('hm <tool_call>{"name": "get_weather", "arguments": {}}</tool_call> ok', True)
    assert (c, t, k[0]["function"]["name"]) == ("ok", "hm", "get_weather")


def test_qwen35_parser_cases():
    """model/parsers/qwen35_test.go restated: reasoning unless switched off, an explicit opening tag is tolerated, a call inside the
    block ends it, a false start of a call mark stays reasoning, a leading closing tag gives content, white space after the block goes."""
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"location": {"type": "string"}}}}}]
    call = "<tool_call><function=get_weather><parameter=location>\nSF\n</parameter></function></tool_call>"

    def run(chunks, think=True, prefill=""):
        p = B.parser_for("qwen3.5", tools, think, prefill)
        out = [p.add(c, i == len(chunks) - 1) for i, c in enumerate(chunks)]
        return "".join(o[0] for o in out), "".join(o[1] for o in out), [k["function"] for o in out for k in o[2]], out

    c, t, k, _ = run(["Need weather lookup" + call])
    assert (c, t, k) == ("", "Need weather lookup", [{"name": "get_weather", "arguments": {"location": "SF"}}])
    c, t, k, _ = run(["Need weather lookup<tool", "_call><function=get_weather><parameter=location>\nSF\n</parameter></function></tool_call>"])
    assert (c, t, len(k)) == ("", "Need weather lookup", 1)
    c, t, k, steps = run(["Need weather lookup<tool_c", "</thi", "nk>"])
    assert (c, t, k) == ("", "Need weather lookup<tool_c", []) and steps[0][1] == "Need weather lookup" and steps[1][1] == "<tool_c"
    assert run(["<think>Let me think</think>Answer."])[:2] == ("Answer.", "Let me think")
    assert run(["I think</think>\n\nDone." + call])[:3] == ("Done.", "I think", [{"name": "get_weather", "arguments": {"location": "SF"}}])
    assert run(["</think>The final answer."])[:2] == ("The final answer.", "")
    assert run(["plain </think> text"], think=False)[:2] == ("plain </think> text", "") and run([" goes on"], prefill="It")[:2] == (" goes on", "")
    assert run(["abc</th", "ink>", "\n\n  ", "def"])[:2] == ("def", "abc") and run(["never closed"])[:2] == ("", "never closed")


def test_cohere_parser_cases():
    """model/parsers/cohere_test.go restated: reasoning up to the end mark, the answer inside text (or legacy response) marks or bare,
    calls as a JSON action list that survives damaged entries, marks split over chunks, continuation of a prefilled answer."""
    def run(chunks, think=None, prefill=""):
        p = B.parser_for("cohere", None, think, prefill)
        out = [p.add(c, i == len(chunks) - 1) for i, c in enumerate(chunks)]
        return "".join(o[0] for o in out), "".join(o[1] for o in out), [k for o in out for k in o[2]]

    assert run(["Let me think", " about this.<|END_THINKING|>", "<|START_TEXT|>Hello", " world!<|END_TEXT|>"]) == ("Hello world!", "Let me think about this.", [])
    assert run(["think<|END_TH", "INKING|><|STAR", "T_TEXT|>ans", "wer<|END_", "TEXT|>"])[:2] == ("answer", "think")
    c, t, k = run(["plan<|END_THINKING|><|START_ACTION|>[\n", '    {"tool_call_id": "0", "tool_name": "get_weather", "parameters": {"city": "Paris"}},',
                   '    {"tool_call_id": "1", "tool_name": "get_time", "parameters": {}}', "\n]<|END_ACTION|>"])
    assert (c, t) == ("", "plan") and [x["function"]["name"] for x in k] == ["get_weather", "get_time"] and k[0]["function"]["arguments"] == {"city": "Paris"} and k[1]["id"] == "1"
    assert run(["<|START_TEXT|>direct answer<|END_TEXT|>"], think=False)[:2] == ("direct answer", "")
    assert run(["thought<|END_THINKING|>", "Just plain text", " output"])[:2] == ("Just plain text output", "thought")
    assert run(["t<|END_THINKING|><|START_TEXT|>answer<|END_OF_TURN_TOKEN|>"])[0] == "answer"
    assert run([" continued<|END_TEXT|>"], prefill="partial")[:2] == (" continued", "")
    k = run(["plan<|END_THINKING|><|START_ACTION|>[\n", '    {"tool_call_id": "0", "tool_name": "set_alarm", "parameters": {"time": 15:30}},',
             '    {"tool_call_id": "1", "tool_name": "get_weather", "parameters": {"city": "Oslo"}}', "\n]<|END_ACTION|>"])[2]
    assert [x["function"]["name"] for x in k] == ["get_weather"]
    k = run(["<|END_THINKING|><|START_ACTION|>[", '{"tool_call_id": "0", "tool_name": "a", "parameters": {}}',
             '{"tool_call_id": "1", "tool_name": "b", "parameters": {"x": "{not json}"}}', "]<|END_ACTION|>"])[2]
    assert [x["function"]["name"] for x in k] == ["a", "b"] and k[1]["function"]["arguments"] == {"x": "{not json}"}
    assert run(["x<|END_THINKING|><|START_ACTION|>[!!!]<|END_ACTION|>"])[2] == []
    assert run(["plan<|END_THINKING|>", "<|START_RESPONSE|>Hello", " there<|END_RESPONSE|>"])[:2] == ("Hello there", "plan")
    for chunk in ("<|START_RESPONSE|>The answer is 42.", "<|TOOL_PLAN|>I should call the tool.", "Just plain text."):
        p = B.parser_for("cohere")
        p.add("x<|END_THINKING|>", False)
        assert p.add(chunk, False)[0] != ""                      # streams before the generation ends
    assert run(["t<|END_THINKING|><|START_TEXT|>hi<|END_TEXT|><|END_OF_TURN_TOKEN|>"])[:2] == ("hi", "t")
    assert run(["t<|END_THINKING|>plain answer<|END_OF_TURN_TOKEN|>"])[0] == "plain answer"


def test_laguna_parser_cases():
    """model/parsers/laguna_test.go, restated: the three spellings of a call body, names mapped to the offered tool, reasoning only
    on request and ended by a call, a repeated closing tag dropped, a continued answer, white space around the answer."""
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"location": {"type": "string"}, "days": {"type": "integer"}}}}}]
    reader = [{"type": "function", "function": {"name": "read", "parameters": {"type": "object", "properties": {"path": {"type": "string"}}}}}]

    def run(name, text, tools=tools, think=None, prefill=""):
        outs = []
        for chunks in ([text], _cut(text, 1), _cut(text, 7)):
            p = B.parser_for(name, tools, think, prefill)
            content = thinking = ""
            calls = []
            for i, ch in enumerate(chunks):
                c, t, k = p.add(ch, i == len(chunks) - 1)
                content, thinking, calls = content + c, thinking + t, calls + k
            outs.append((content, thinking, [(k["function"]["name"], k["function"]["arguments"]) for k in calls]))
        assert outs[0] == outs[1] == outs[2], text
        return outs[0]

    pairs = "<tool_call>get_weather\n<arg_key>location</arg_key>\n<arg_value>Paris</arg_value>\n<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n</tool_call>"
    assert run("laguna", pairs) == ("", "", [("get_weather", {"location": "Paris", "days": 3})])
    assert run("laguna", '<tool_call>get_weather\n{"location":"San Francisco"}</tool_call>') == ("", "", [("get_weather", {"location": "San Francisco"})])
    assert run("laguna", '<tool_call>\n{"name":"read_file","arguments":{"path":"./go.mod"}}\n</tool_call>', tools=reader) == ("", "", [("read", {"path": "./go.mod"})])
    assert run("laguna", '<tool_call>\n{"name":"read_file","arguments":{"path":"x"}}\n</tool_call>')[2] == [("read_file", {"path": "x"})]      # no such tool offered: as written
    assert run("laguna", "I should check.</think>\n\n" + pairs, think=True) == ("", "I should check.", [("get_weather", {"location": "Paris", "days": 3})])
    assert run("laguna", "Let me look." + pairs, think=True)[1:] == ("Let me look.", [("get_weather", {"location": "Paris", "days": 3})])
    assert run("laguna", "<think>\nhm\n</think>\nfine", think=True) == ("fine", "hm", [])
    assert run("laguna", "Just an answer", think=True) == ("", "Just an answer", [])             # the prompt ended inside the block
    for think in (None, False):
        assert run("laguna", "</think>\n\n  Hello there  \n", think=think) == ("Hello there", "", [])
        assert run("laguna", "Plain answer", think=think, tools=None) == ("Plain answer", "", [])
    assert run("laguna", " continues here", think=True, prefill="It") == ("continues here", "", [])
    assert run("poolside-v1", "thinking</think>answer", think=True, prefill="It") == ("answer", "thinking", [])
    assert run("laguna", "ok <tool_call>never closed", think=None) == ("ok<tool_call>never closed", "", [])


def _glimmer_tool(name, props=None):
    return {"type": "function", "function": {"name": name, "parameters": {"type": "object", "properties": props or {}}}}


def _atem(name, params=""):
    return f'<atem:function_calls>\n<atem:invoke name="{name}">\n{params}</atem:invoke>\n</atem:function_calls>'


def _glimmer_run(text, tools=None, think=None, cuts=None):
    """Every two-chunk split of ``text`` (or the given cut points) gives the same result; returns it."""
    outs = set()
    for split in (range(len(text) + 1) if cuts is None else cuts):
        p = B.parser_for("glimmer", tools, think)
        content = thinking = ""
        calls = []
        for i, ch in enumerate((text[:split], text[split:])):
            c, t, k = p.add(ch, i == 1)
            content, thinking, calls = content + c, thinking + t, calls + k
        outs.add((content, thinking, json.dumps([(k["function"]["name"], k["function"]["arguments"]) for k in calls])))
    assert len(outs) == 1, outs
    c, t, k = outs.pop()
    return c, t, [tuple(x) for x in json.loads(k)]


def test_glimmer_parser_cases():
    """model/parsers/glimmer_test.go, restated: addressed messages, reasoning on and off, typed call values, mark text inside a
    value, several messages at every split point, the repeated name space, a call without an address, text that only looks like one."""
    assert _glimmer_run(" to=user<|message|>Hello") == ("Hello", "", [])
    assert _glimmer_run(" to=self<|message|>Check the facts.") == ("", "Check the facts.", [])
    both = " to=self<|message|>Check the facts.<|eom|><|start|>assistant to=user<|message|>Answer<|eot|>"
    assert _glimmer_run(both, think=False) == ("Answer", "", [])
    assert _glimmer_run(both) == ("Answer", "Check the facts.", [])
    assert _glimmer_run(" to=self<|message|>Think<|start|>assistant to=user<|message|>Answer") == ("Answer", "Think", [])      # no end mark
    tool = _glimmer_tool("tools.run", {"text": {"type": "string"}, "count": {"type": "integer"}, "enabled": {"type": "boolean"}, "items": {"type": "array"},
                                       "config": {"type": "object"}, "choice": {"anyOf": [{"type": "null"}, {"type": "string"}]}})
    params = ('<atem:parameter name="text"> keep  spaces </atem:parameter>\n<atem:parameter name="count">3</atem:parameter>\n'
              '<atem:parameter name="enabled">true</atem:parameter>\n<atem:parameter name="items">["one", "two"]</atem:parameter>\n'
              '<atem:parameter name="config">{"mode":"fast"}</atem:parameter>\n<atem:parameter name="choice">null</atem:parameter>\n')
    want = {"text": " keep  spaces ", "count": 3, "enabled": True, "items": ["one", "two"], "config": {"mode": "fast"}, "choice": None}
    assert _glimmer_run(" to=tools.run<|message|>" + _atem("tools.run", params), [tool], cuts=(0, 40, 200)) == ("", "", [("tools.run", want)])
    assert _glimmer_run(" to=tools.tools.run<|message|>" + _atem("tools.run", params), [tool], cuts=(0,))[2] == [("tools.run", want)]     # name space said twice
    echo = _glimmer_tool("echo", {"text": {"type": "string"}})
    value = "literal <|eot|> and <|start|>assistant to=user<|message|> text"
    got = _glimmer_run(" to=echo<|message|>" + _atem("echo", f'<atem:parameter name="text">{value}</atem:parameter>\n') + "<|eot|>", [echo])
    assert got == ("", "", [("echo", {"text": value})])
    first, second = _glimmer_tool("first", {"x": {"type": "integer"}}), _glimmer_tool("second")
    run = (" to=self<|message|>Think<|eom|><|start|>assistant to=first<|message|>" + _atem("first", '<atem:parameter name="x">1</atem:parameter>\n')
           + "<|eom|><|start|>assistant to=second<|message|>" + _atem("second") + "<|eot|>")
    assert _glimmer_run(run, [first, second]) == ("", "Think", [("first", {"x": 1}), ("second", {})])
    assert _glimmer_run(" to=user<|message|>" + _atem("echo", '<atem:parameter name="text">hi</atem:parameter>\n') + "<|eot|>", [echo]) == ("", "", [("echo", {"text": "hi"})])
    looks = " to=user<|message|>Use " + _atem("echo") + " like this.<|eot|>"
    assert _glimmer_run(looks, [echo]) == ("Use " + _atem("echo") + " like this.", "", [])
    assert _glimmer_run(" to=nobody<|message|>Hi<|eot|>", [echo]) == ("Hi", "", [])                 # an undeclared recipient reads as the answer
    with pytest.raises(ValueError):
        B.parser_for("glimmer", [first, second]).add(" to=first<|message|>" + _atem("second") + "<|eot|>", True)
    with pytest.raises(ValueError):
        B.parser_for("glimmer", [first]).add(" to=first<|message|><atem:function_calls>oops<|eot|>", True)


def test_gemma4_argument_notation_as_json():
    """model/parsers/gemma4_test.go (TestGemma4ArgsToJSON), as data: delimited strings, bare keys, nesting, strings that look like keys."""
    rows = DATA["gemma4_args"]
    assert len(rows) >= 25
    for c in rows:
        assert json.loads(B.gemma4_args_to_json(c["input"])) == json.loads(c["expected"]), c["case"]
    # the stream may end inside a call; what a model adds behind a call goes; reasoning is parsed but withheld unless asked for
    p = B.parser_for("gemma4", None, None)
    assert p.add('<|channel>thought\nhm<channel|>ok <|tool_call>call:f{a:<|"|>x<|"|>,n:2}', True) == ("ok", "", [{"function": {"name": "f", "arguments": {"a": "x", "n": 2}}}])
    p = B.parser_for("gemma4", None, True, "", True)                # after tool results a reasoning request goes on inside the channel
    assert p.add("more thought<channel|>done<tool_call|><|tool_response>", True) == ("done", "more thought", [])
    p = B.parser_for("gemma4-no-thinking", None, True)
    assert p.add("<|channel>thought\nhm<channel|>ok", True) == ("ok", "", [])
