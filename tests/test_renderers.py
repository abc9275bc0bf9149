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
        r.image_tags = case["image_tags"]
    if "current_date" in case:
        r.current_date = case["current_date"]
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
    assert covered >= set(R.DIALECTS) - {"olmo3.1", "qwen3.5", "qwen3.8", "ornith", "cohere", "gemma4-small", "gemma4-large"}   # these have tests of their own below
    for name in set(R.DIALECTS) - {"qwen3.8"}:
        assert isinstance(R.renderer_for(name).render([], None, None), str)
    assert R.renderer_for("olmo3.1").render([{"role": "user", "content": "hi"}]).startswith("<|im_start|>system\nYou are Olmo, a helpful AI assistant built by Ai2.")
    assert R.renderer_for("nope") is None and R.renderer_for(None) is None


def test_glm_ocr_turns_reasoning_switch_and_tools():
    """model/renderers/glmocr.go:27-107 beyond the image cases of its own test table: the stored reasoning of an assistant turn, calls
    and their results, a system message in place, the ``/nothink`` nudge and the empty block when reasoning is switched off."""
    r = R.renderer_for("glm-ocr")
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "read it"},
            {"role": "assistant", "content": " ok ", "thinking": " plan ", "tool_calls": [{"function": {"name": "ocr", "arguments": {"page": 2, "lang": "en"}}}]},
            {"role": "tool", "content": "text A"}, {"role": "tool", "content": "text B"}, {"role": "user", "content": "and now?"}]
    got = r.render(msgs, None, False)
    assert got == ("[gMASK]<sop><|system|>\nBe brief.\n<|user|>\nread it/nothink<|assistant|>\n<think>plan</think>\nok\n<tool_call>ocr"
                   "<arg_key>page</arg_key><arg_value>2</arg_value><arg_key>lang</arg_key><arg_value>en</arg_value></tool_call>\n"
                   "<|observation|>\n<tool_response>\ntext A\n</tool_response>\n\n<tool_response>\ntext B\n</tool_response>\n"
                   "<|user|>\nand now?/nothink<|assistant|>\n<think></think>\n")
    assert r.render(msgs[1:2], None, None) == "[gMASK]<sop><|user|>\nread it<|assistant|>\n"
    tools = [{"type": "function", "function": {"name": "ocr", "description": "read a page", "parameters": {"type": "object", "properties": {"page": {"type": "integer"}}}}}]
    head = r.render(msgs[1:2], tools, True)
    assert head.startswith("[gMASK]<sop><|system|>\n# Tools\n\nYou may call one or more functions") and '"name": "ocr"' in head
    assert head.endswith("<arg_value>{arg-value-2}</arg_value>...</tool_call><|user|>\nread it<|assistant|>\n")
    from ollama_b200.text.builtin import parser_for
    p = parser_for("glm-ocr", tools, None)
    content, thinking, calls = p.add("done <tool_call>ocr<arg_key>page</arg_key><arg_value>3</arg_value></tool_call>", True)
    assert content.strip() == "done" and thinking == "" and calls[0]["function"] == {"name": "ocr", "arguments": {"page": 3}}


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


def test_qwen35_family():
    """Cases of model/renderers/qwen35_test.go, qwen38_test.go and ornith_test.go restated: XML calls under JSON declarations, the
    system text after the tool section, reasoning kept only after the last question (3.5) or on every stored turn (3.8, ornith),
    merged instructions and the reasoning-effort sentence of 3.8, its refusals."""
    tc = lambda n, **a: {"function": {"name": n, "arguments": a}}   # noqa: E731
    XH, LOW = R._QWEN38_EFFORT["high"], R._QWEN38_EFFORT["low"]
    U = lambda c: f"<|im_start|>user\n{c}<|im_end|>\n"              # noqa: E731
    CUE = "<|im_start|>assistant\n<think>\n"
    r35, r38 = R.Qwen35(image_tags=False), R.Qwen35(always_block=True, effort=True, image_tags=False)
    tools = [{"type": "function", "function": {"name": n, "description": d, "parameters": {"type": "object", "required": ["city"], "properties": {"city": {"type": "string"}}}}}
             for n, d in (("get_weather", "Get weather"), ("get_uv", "Get UV index"))]
    msgs = [{"role": "system", "content": "You are a helpful assistant."}, {"role": "user", "content": "Run add and multiply."},
            {"role": "assistant", "content": "I'll run both now.", "thinking": "Need to call add and multiply.", "tool_calls": [tc("add", a=2, b=3), tc("multiply", x=4, y=5)]},
            {"role": "tool", "content": "5"}, {"role": "tool", "content": "20"}, {"role": "user", "content": "Summarize the results."}]
    got = r35.render(msgs, tools)
    assert "Need to call add" not in got and got.index("# Tools") < got.index("You are a helpful assistant.") and got.endswith(CUE)
    assert ("<tool_call>\n<function=add>\n<parameter=a>\n2\n</parameter>\n<parameter=b>\n3\n</parameter>\n</function>\n</tool_call>\n<tool_call>\n<function=multiply>\n"
            "<parameter=x>\n4\n</parameter>\n<parameter=y>\n5\n</parameter>\n</function>\n</tool_call>") in got
    assert "<|im_start|>user\n<tool_response>\n5\n</tool_response>\n<tool_response>\n20\n</tool_response><|im_end|>" in got
    msgs = [{"role": "user", "content": "Plan a picnic."}, {"role": "assistant", "content": "Checking weather first.", "thinking": "Need weather.", "tool_calls": [tc("get_weather", city="Paris")]},
            {"role": "tool", "content": "22C"}]
    assert ("<|im_start|>assistant\n<think>\nNeed weather.\n</think>\n\nChecking weather first.\n\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n"
            "</function>\n</tool_call><|im_end|>") in r35.render(msgs, tools)
    assert r35.render([{"role": "user", "content": "Write two words."}, {"role": "assistant", "thinking": "Keep it short.", "content": "Hello world"}]) == \
        U("Write two words.") + "<|im_start|>assistant\n<think>\nKeep it short.\n</think>\n\nHello world"
    assert r35.render([{"role": "user", "content": "hello"}], None, False).endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    # reasoning left inside stored content by an older client is moved into the block (3.5 only)
    assert "<think>\nplan\n</think>\n\nAnswer" in r35.render([{"role": "user", "content": "q"}, {"role": "assistant", "content": "<think>plan</think>\nAnswer"}])
    # 3.8
    sys = lambda body: f"<|im_start|>system\n{body}<|im_end|>\n"    # noqa: E731
    assert r38.render([{"role": "user", "content": "Hello"}]) == sys(XH) + U("Hello") + CUE
    assert r38.render([{"role": "developer", "content": "Use Go."}, {"role": "user", "content": "Hello"}]) == sys(XH + "\n\nUse Go.") + U("Hello") + CUE
    flow = [{"role": "system", "content": "Base policy."}, {"role": "user", "content": "Base question"}, {"role": "assistant", "content": "Base answer"},
            {"role": "system", "content": "Request policy."}, {"role": "user", "content": "Current question"}]
    assert r38.render(flow) == (sys(XH + "\n\nBase policy.\n\nRequest policy.") + U("Base question") + "<|im_start|>assistant\n<think>\n\n</think>\n\nBase answer<|im_end|>\n"
                                + U("Current question") + CUE)
    assert r38.render([{"role": "system", "content": " Be concise. \n"}, {"role": "user", "content": "Hello"}], None, True) == sys("Be concise.") + U("Hello") + CUE
    assert r38.render([{"role": "user", "content": "Hello"}], None, "low") == sys(LOW) + U("Hello") + CUE
    assert r38.render([{"role": "user", "content": "Hello"}], None, False) == U("Hello") + "<|im_start|>assistant\n<think>\n\n</think>\n\n"
    kept = [{"role": "user", "content": "First"}, {"role": "assistant", "thinking": "Plan", "content": "<think>literal</think>\nAnswer"}, {"role": "user", "content": "Next"}]
    assert r38.render(kept) == sys(XH) + U("First") + "<|im_start|>assistant\n<think>\nPlan\n</think>\n\n<think>literal</think>\nAnswer<|im_end|>\n" + U("Next") + CUE
    got = r38.render([{"role": "developer", "content": "Use tools when requested."}, {"role": "user", "content": "Check the weather."}], tools, True)
    assert got.startswith("<|im_start|>system\n# Tools\n\nYou have access to the following functions:\n\n<tools>\n" + R.go_json(R.tool_schema(tools[0]), spaced=True) + "\n")
    assert got.endswith("</IMPORTANT>\n\nUse tools when requested.<|im_end|>\n" + U("Check the weather.") + CUE)
    got = r38.render([{"role": "user", "content": "Weather?"}, {"role": "assistant", "thinking": "Need current data.", "content": "I'll check.", "tool_calls": [tc("get_weather", city="Montréal")]},
                      {"role": "tool", "content": '{"temp": 18}'}], tools, True)
    assert got.endswith(U("Weather?") + "<|im_start|>assistant\n<think>\nNeed current data.\n</think>\n\nI'll check.\n\n<tool_call>\n<function=get_weather>\n<parameter=city>\nMontréal\n"
                        "</parameter>\n</function>\n</tool_call><|im_end|>\n<|im_start|>user\n<tool_response>\n{\"temp\": 18}\n</tool_response><|im_end|>\n" + CUE)
    assert r38.render([{"role": "user", "content": "Describe this.", "images": ["x"]}], None, False).startswith(U("<|vision_start|><|image_pad|><|vision_end|>Describe this."))
    for bad, why in (([], "no messages provided"), ([{"role": "system", "content": "Hello"}], "no user query"),
                     ([{"role": "system", "images": ["x"]}, {"role": "user", "content": "Hello"}], "cannot contain images")):
        with pytest.raises(R.RenderError, match=why):
            r38.render(bad)
    with pytest.raises(R.RenderError):
        r38.render([{"role": "user", "content": "x"}], None, "extreme")
    # ornith: every stored assistant turn carries a block, also with thinking switched off
    orn = R.renderer_for("ornith")
    got = orn.render([{"role": "user", "content": "a"}, {"role": "assistant", "content": "b"}, {"role": "user", "content": "c"}], None, False)
    assert "<|im_start|>assistant\n<think>\n\n</think>\n\nb<|im_end|>" in got and got.endswith("<think>\n\n</think>\n\n")


def test_cohere_renderer():
    """model/renderers/cohere_test.go restated (expectations there come from the checkpoint's own Jinja template)."""
    r = R.renderer_for("cohere")
    T0, T1 = "<|START_OF_TURN_TOKEN|>", "<|END_OF_TURN_TOKEN|>"
    no_tools = f"{T0}<|SYSTEM_TOKEN|><|START_TEXT|># Available Tools\n```json\n[\n\n\n\n]\n```<|END_TEXT|>{T1}"
    user = lambda c: f"{T0}<|USER_TOKEN|><|START_TEXT|>{c}<|END_TEXT|>{T1}"      # noqa: E731
    assert r.render([{"role": "user", "content": "USERMSG"}]) == no_tools + user("USERMSG") + f"{T0}<|CHATBOT_TOKEN|><|START_THINKING|>"
    got = r.render([{"role": "system", "content": "DEVPREAMBLE"}, {"role": "user", "content": "Q1"}, {"role": "assistant", "content": "A1", "thinking": "THINK1"},
                    {"role": "user", "content": "Q2"}])
    assert got == (f"{T0}<|SYSTEM_TOKEN|><|START_TEXT|>DEVPREAMBLE\n\n\n\n# Available Tools\n```json\n[\n\n\n\n]\n```<|END_TEXT|>{T1}" + user("Q1")
                   + f"{T0}<|CHATBOT_TOKEN|><|START_THINKING|>THINK1<|END_THINKING|><|START_TEXT|>A1<|END_TEXT|>{T1}" + user("Q2") + f"{T0}<|CHATBOT_TOKEN|><|START_THINKING|>")
    assert r.render([{"role": "user", "content": "Q"}], None, False).endswith(f"{T0}<|CHATBOT_TOKEN|><|START_THINKING|><|END_THINKING|>")
    tools = [{"type": "function", "function": {"name": "get_weather", "description": "Get weather",
                                               "parameters": {"type": "object", "required": ["city"], "properties": {"city": {"type": "string"}}}}}]
    got = r.render([{"role": "user", "content": "weather in Paris?"},
                    {"role": "assistant", "thinking": "I should call the tool", "tool_calls": [{"id": "call_x", "function": {"name": "get_weather", "arguments": {"city": "Paris"}}}]},
                    {"role": "tool", "tool_call_id": "call_x", "content": "15C sunny"}, {"role": "user", "content": "thanks"}], tools)
    assert ('# Available Tools\n```json\n[\n\n    {"name": "get_weather", "description": "Get weather", "parameters": {"type": "object", "required": ["city"], '
            '"properties": {"city": {"type": "string"}}}, "responses": null}\n\n\n]\n```') in got
    assert (f'{T0}<|CHATBOT_TOKEN|>\n            \n                <|START_THINKING|>I should call the tool<|END_THINKING|><|START_ACTION|>[\n\n    '
            f'{{"tool_call_id": "0", "tool_name": "get_weather", "parameters": {{"city": "Paris"}}}}\n\n]<|END_ACTION|>{T1}') in got
    assert (f'{T0}<|SYSTEM_TOKEN|><|START_TOOL_RESULT|>[\n    {{\n        "tool_call_id": "0",\n        "results": {{\n\n            \n            "0": {{"content": "15C sunny"}}'
            f'\n\n        }},\n        "is_error": null\n    }}\n\n]<|END_TOOL_RESULT|>{T1}') in got
    got = r.render([{"role": "user", "content": "go"},
                    {"role": "assistant", "tool_calls": [{"id": "a", "function": {"name": "t1", "arguments": {}}}, {"id": "b", "function": {"name": "t2", "arguments": {"x": 1}}}]},
                    {"role": "tool", "tool_call_id": "a", "content": "r1"}, {"role": "tool", "tool_call_id": "b", "content": "r2"}])
    assert ('<|START_ACTION|>[\n\n    {"tool_call_id": "0", "tool_name": "t1", "parameters": {}},\n\n    {"tool_call_id": "1", "tool_name": "t2", "parameters": {"x": 1}}\n\n]'
            '<|END_ACTION|>') in got
    assert ('<|START_TOOL_RESULT|>[\n    {\n        "tool_call_id": "0",\n        "results": {\n\n            \n            "0": {"content": "r1"}\n\n        },\n'
            '        "is_error": null\n    },\n    {\n        "tool_call_id": "1",\n        "results": {\n\n            \n            "0": {"content": "r2"}\n\n        },\n'
            '        "is_error": null\n    }\n\n]<|END_TOOL_RESULT|>') in got
    assert r.render([{"role": "user", "content": "Q"}, {"role": "Chatbot", "content": "partial"}]).endswith(f"{T0}<|CHATBOT_TOKEN|><|START_TEXT|>partial")


def test_glimmer_images_call_values_strength_and_result_names():
    """model/renderers/glimmer_test.go, restated."""
    g = R.renderer_for("glimmer")
    g.image_tags = False
    assert "<|start|>user<|message|><|patch|>Describe.<|eot|>" in g.render([{"role": "user", "content": "Describe.", "images": ["aQ=="]}])
    tagged = R.renderer_for("glimmer").render([{"role": "user", "content": "First.", "images": ["aQ=="]}, {"role": "assistant", "content": "Done."},
                                               {"role": "user", "content": "Compare.", "images": ["ag==", "aw=="]}])
    assert ("<|start|>user<|message|>[img-0] First.<|eot|><|start|>assistant to=user<|message|>Done.<|eot|>"
            "<|start|>user<|message|>[img-1][img-2] Compare.<|eot|>") in tagged
    args = {"text": "keep  spaces", "count": 3, "enabled": True, "fallback": None, "items": ["one", "two"], "config": {"mode": "fast"}}
    got = g.render([{"role": "user", "content": "Run it."}, {"role": "assistant", "tool_calls": [{"function": {"name": "tools.run", "arguments": args}}]}])
    assert ('<atem:function_calls>\n<atem:invoke name="tools.run">\n<atem:parameter name="text">keep  spaces</atem:parameter>\n'
            '<atem:parameter name="count">3</atem:parameter>\n<atem:parameter name="enabled">true</atem:parameter>\n'
            '<atem:parameter name="fallback">null</atem:parameter>\n<atem:parameter name="items">["one", "two"]</atem:parameter>\n'
            '<atem:parameter name="config">{"mode": "fast"}</atem:parameter>\n</atem:invoke>\n</atem:function_calls>') in got
    for think, want in ((None, "high"), (True, "high"), (False, "none"), ("medium", "medium")):
        assert f"Reasoning strength: {want}." in g.render([{"role": "user", "content": "Hello"}], None, think)
    got = g.render([{"role": "assistant", "tool_calls": [{"id": "call_1", "function": {"name": "get_weather", "arguments": {}}}]},
                    {"role": "tool", "tool_call_id": "call_1", "content": '{"temp":65}'}, {"role": "tool", "tool_call_id": "missing", "content": "not found"}])
    assert '<|start|>tool get_weather<|message|><tool_output name="get_weather">\n{"temp":65}\n</tool_output><|eot|>' in got
    assert '<|start|>tool missing<|message|><tool_output name="missing">\nnot found\n</tool_output><|eot|>' in got
    import datetime
    days = {datetime.date.today().isoformat(), (datetime.date.today() - datetime.timedelta(days=1)).isoformat()}      # the day may turn in between
    assert any(f"Current date: {d}." in g.render([{"role": "user", "content": "x"}]) for d in days)


def test_gemma4_variants_and_turns_that_continue():
    """model/renderers/gemma4_reference_test.go, the tables besides the main one: the large checkpoints' empty thought channel in the
    cue (not when the request reasons), and a run of assistant messages with a call and its result rendered as one model turn."""
    hello = [{"role": "user", "content": "Hello"}]
    base = "<bos><|turn>user\nHello<turn|>\n<|turn>model\n"
    assert R.renderer_for("gemma4").render(hello) == R.renderer_for("gemma4-small").render(hello) == base
    assert R.renderer_for("gemma4-large").render(hello) == base + "<|channel>thought\n<channel|>"
    assert R.renderer_for("gemma4-large").render(hello, None, True) == "<bos><|turn>system\n<|think|>\n<turn|>\n<|turn>user\nHello<turn|>\n<|turn>model\n"
    msgs = [{"role": "user", "content": "Use the tool"}, {"role": "assistant", "content": "First."},
            {"role": "assistant", "content": "Checking.", "tool_calls": [{"function": {"name": "bash", "arguments": {"command": None}}}]},
            {"role": "tool", "tool_name": "bash", "content": "done"}, {"role": "assistant", "content": "Done."}, {"role": "user", "content": "Next"}]
    tool = [{"type": "function", "function": {"name": "bash", "description": "Run", "parameters": {"type": "object", "required": ["command"],
                                                                                                    "properties": {"command": {"type": "string", "description": "Cmd"}}}}}]
    q = '<|"|>'
    decl = (f"<|tool>declaration:bash{{description:{q}Run{q},parameters:{{properties:{{command:{{description:{q}Cmd{q},type:{q}STRING{q}}}}},"
            f"required:[{q}command{q}],type:{q}OBJECT{q}}}}}<tool|>")
    want = ("<bos><|turn>system\n" + decl + "<turn|>\n<|turn>user\nUse the tool<turn|>\n<|turn>model\nFirst.<|tool_call>call:bash{command:null}<tool_call|>"
            f"<|tool_response>response:bash{{value:{q}done{q}}}<tool_response|>Checking.Done.<turn|>\n<|turn>user\nNext<turn|>\n<|turn>model\n")
    assert R.renderer_for("gemma4").render(msgs, tool) == want
    assert R.renderer_for("gemma4-large").render(msgs, tool) == want + "<|channel>thought\n<channel|>"
    # a union of bare types written as anyOf reads as a type list
    union = [{"type": "function", "function": {"name": "f", "description": "d", "parameters": {"type": "object", "properties": {"v": {"anyOf": [{"type": "string"}, {"type": "null"}]}}}}}]
    assert f"v:{{type:{q}['STRING', 'NULL']{q}}}" in R.renderer_for("gemma4").render(hello, union)
