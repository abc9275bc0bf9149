"""Built-in prompt renderers on the reference's own cases.

``tests/data/renderer_cases.json`` restates the tables of the reference's renderer tests (model/renderers/*_test.go: messages,
tools and think value of every case with the prompt it expects) as data, so that the comparison needs no checkout of the
reference.  ``source`` and ``case`` name the table and the row a case comes from.
"""
import json
import os

import pytest

from ollama_b200.text import renderers as R

with open(os.path.join(os.path.dirname(__file__), "data", "renderer_cases.json"), encoding="utf-8") as _f:
    CASES = json.load(_f)


def _renderer(case):
    r = R.renderer_for(case["renderer"])
    if "image_tags" in case:
        r = R.Qwen3VL(r.thinking, image_tags=case["image_tags"])
    return r


@pytest.mark.parametrize("name", sorted({c["renderer"] for c in CASES}))
def test_renderer_reproduces_the_reference_prompts(name):
    mine = [c for c in CASES if c["renderer"] == name]
    assert mine
    for c in mine:
        got = _renderer(c).render(c["messages"], c.get("tools"), c.get("think"))
        assert got == c["expected"], (c["source"], c["case"])


def test_every_registered_renderer_has_cases_and_renders_an_empty_conversation():
    covered = {c["renderer"] for c in CASES}
    assert covered >= set(R.DIALECTS) - {"olmo3.1"}
    for name in R.DIALECTS:
        assert isinstance(R.renderer_for(name).render([], None, None), str)
    assert R.renderer_for("olmo3.1").render([{"role": "user", "content": "hi"}]).startswith("<|im_start|>system\nYou are Olmo, a helpful AI assistant built by Ai2.")
    assert R.renderer_for("nope") is None and R.renderer_for(None) is None


def test_conversation_normal_form():
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "q", "images": ["a", "b"]},
            {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "f", "arguments": {"x": 1}}}, {"function": {"name": "g", "arguments": {}}}]},
            {"role": "tool", "content": "1"}, {"role": "tool", "content": "2", "tool_name": "other"}, {"role": "tool", "content": "3", "tool_name": "h"},
            {"role": "system", "content": "late"}, {"role": "user", "content": "again", "images": ["c"]}, {"role": "assistant", "content": "par"}]
    c = R.Conversation(msgs)
    assert c.system_text == "S" and [t.role for t in c.turns] == ["user", "assistant", "tool", "system", "user", "assistant"]
    assert c.turns[2].results == [("f", "1"), ("g", "2"), ("h", "3")]            # by position among the calls first, by the message's own name after that
    assert c.turns[4].first_image == 2 and c.continued is c.turns[-1] and c.last_user() == 4
    assert R.Conversation(msgs, system="first").system_text == "S" and "system" not in [t.role for t in R.Conversation(msgs, system="first").turns]
    assert R.Conversation(msgs, system="join").system_text == "S\n\nlate"
    assert R.Conversation(msgs, system="inline").turns[0].role == "system"
    assert R.Conversation(msgs[:3]).continued is None                                # an assistant turn with calls is not continued


def test_json_in_the_reference_encoders_spelling():
    assert R.go_json({"b": 1.0, "a": "<x>&"}) == '{"b":1,"a":"\\u003cx\\u003e\\u0026"}'
    assert R.go_json({"b": [1, {"d": 2, "c": 3}]}, spaced=True) == '{"b": [1, {"d": 2, "c": 3}]}'
    assert R.args_json({"z": {"b": 1, "a": 2}, "a": 0}) == '{"z":{"a":2,"b":1},"a":0}'
    tool = {"function": {"parameters": {"properties": {"p": {"description": "d", "type": ["string"], "enum": ["a"]}}, "required": ["p"], "type": "object"},
                         "description": "D", "name": "n"}, "type": "function"}
    assert R.go_json(R.tool_schema(tool)) == ('{"type":"function","function":{"name":"n","description":"D","parameters":{"type":"object","required":["p"],'
                                              '"properties":{"p":{"type":"string","description":"d","enum":["a"]}}}}}')
    assert R.image_tagged("look [img] and", 2, 3) == "[img-4] look [img-3] and" and R.image_tagged("x", 0, 0) == "x" and R.image_tagged("[img-0] x", 1, 5) == "[img-0] x"
