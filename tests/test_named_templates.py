"""Named chat layouts: Go-template text generated from the layout table, detection from Jinja chat templates, create-time use.

The expected prompts restate the golden files of the reference's template tests (template/testdata/<layout>/<case>) for the
conversation system / user / assistant / user; the full set of golden files and of recognised Jinja templates is checked as
well when OLLAMA_REFERENCE_DIR points at a checkout of the reference.
"""
import json
import os

import pytest

from ollama_b200.text import named
from ollama_b200.text.template import Template

CONV = [("system", "You are a helpful assistant."), ("user", "Hello, how are you?"), ("assistant", "I'm doing great. How can I help you today?"),
        ("user", "I'd like to show off how chat templating works!")]
S, U1, A1, U2 = (c for _, c in CONV)
GOLDEN = {
    "chatml": f"<|im_start|>system\n{S}<|im_end|>\n<|im_start|>user\n{U1}<|im_end|>\n<|im_start|>assistant\n{A1}<|im_end|>\n<|im_start|>user\n{U2}<|im_end|>\n<|im_start|>assistant\n",
    "llama3-instruct": f"<|start_header_id|>system<|end_header_id|>\n\n{S}<|eot_id|><|start_header_id|>user<|end_header_id|>\n\n{U1}<|eot_id|>"
                       f"<|start_header_id|>assistant<|end_header_id|>\n\n{A1}<|eot_id|><|start_header_id|>user<|end_header_id|>\n\n{U2}<|eot_id|>"
                       f"<|start_header_id|>assistant<|end_header_id|>\n\n",
    "llama2-chat": f"[INST] <<SYS>>\n{S}\n<</SYS>>\n\n{U1} [/INST] {A1}</s><s>[INST] <<SYS>><</SYS>>\n\n{U2} [/INST]",
    "mistral-instruct": f"[INST] {S}\n\n{U1}[/INST] {A1}</s>[INST] {U2}[/INST]",
    "gemma-instruct": f"<start_of_turn>user\n{S}\n{U1}<end_of_turn>\n<start_of_turn>model\n{A1}<end_of_turn>\n<start_of_turn>user\n{U2}<end_of_turn>\n<start_of_turn>model\n",
    "gemma3-instruct": f"<start_of_turn>user\n{S}\n\n{U1}<end_of_turn>\n<start_of_turn>model\n{A1}<end_of_turn>\n<start_of_turn>user\n{U2}<end_of_turn>\n<start_of_turn>model\n\n",
    "phi-3": f"<|system|>\n{S}<|end|>\n<|user|>\n{U1}<|end|>\n<|assistant|>\n{A1}<|end|>\n<|user|>\n{U2}<|end|>\n<|assistant|>\n",
    "zephyr": f"<|system|>\n{S}</s>\n<|user|>\n{U1}</s>\n<|assistant|>\n{A1}</s>\n<|user|>\n{U2}</s>\n<|assistant|>\n",
    "command-r": f"<|START_OF_TURN_TOKEN|><|SYSTEM_TOKEN|>{S}<|END_OF_TURN_TOKEN|><|START_OF_TURN_TOKEN|><|USER_TOKEN|>{U1}<|END_OF_TURN_TOKEN|>"
                 f"<|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>{A1}<|END_OF_TURN_TOKEN|><|START_OF_TURN_TOKEN|><|USER_TOKEN|>{U2}<|END_OF_TURN_TOKEN|>"
                 f"<|END_OF_TURN_TOKEN|><|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>\n",
    "openchat": f"GPT4 Correct System: {S}<|end_of_turn|>GPT4 Correct User: {U1}<|end_of_turn|>GPT4 Correct Assistant: {A1}<|end_of_turn|>"
                f"GPT4 Correct User: {U2}<|end_of_turn|>GPT4 Correct Assistant:",
    "alpaca": f"{S}\n\n### Instruction:\n{U1}\n\n### Response:\n{A1}\n\n### Instruction:\n{U2}\n\n### Response:\n",
    "magicoder": f"{S}\n\n@@ Instruction\n{U1}\n\n@@ Response\n{A1}\n\n@@ Instruction\n{U2}\n\n@@ Response\n",
    "starcoder2-instruct": f"{S}\n\n### Instruction\n{U1}\n\n### Response\n{A1}<|endoftext|>\n\n### Instruction\n{U2}\n\n### Response\n",
    "solar-instruct": f"### System:\n{S}\n\n### User:\n{U1}\n\n### Assistant:\n{A1}</s>\n\n### User:\n{U2}\n\n### Assistant:\n",
    "granite-instruct": f"System:\n{S}\n\nQuestion:\n{U1}\n\nAnswer:\n{A1}\n\nQuestion:\n{U2}\n\nAnswer:\n",
    "chatqa": f"System: {S}\n\nUser: {U1}\n\nAssistant: {A1}\n\nUser: {U2}\n\nAssistant:",
    "falcon-instruct": f"System: {S}\nUser:\n{U1}\nFalcon:\n{A1}\nUser:\n{U2}\nFalcon:\n",
    "vicuna": f"{S}\n\nUSER: {U1}\nASSISTANT: {A1}</s>\nUSER: {U2}\nASSISTANT:",
    "alfred": f"<start_system>{S}<end_message><start_user>{U1}<end_message><start_assistant>{A1}<end_message><start_user>{U2}<end_message><start_assistant>",
    "codellama-70b-instruct": f"Source: system\n\n {S} <step> Source: user\n\n {U1} <step> Source: assistant\n\n {A1} <step> Source: user\n\n {U2} <step> "
                              f"Source: assistant\nDestination: user\n\n ",
}


def _msgs(conv):
    return [{"role": r, "content": c} for r, c in conv]


def test_every_layout_renders_its_golden_prompt():
    assert set(GOLDEN) == set(named.BY_NAME)
    for name, want in GOLDEN.items():
        text, stop = named.named(name)
        assert Template(text).execute(messages=_msgs(CONV)) == want, name
        assert stop, name


def test_a_trailing_assistant_message_is_continued_not_closed():
    t = Template(named.named("chatml")[0])
    got = t.execute(messages=_msgs([("user", "Hi"), ("assistant", "Once upon")]))
    assert got == "<|im_start|>user\nHi<|im_end|>\n<|im_start|>assistant\nOnce upon"
    t = Template(named.named("llama2-chat")[0])
    assert t.execute(messages=_msgs([("user", "Hi"), ("assistant", "Once")])) == "[INST] <<SYS>><</SYS>>\n\nHi [/INST] Once"


def test_levenshtein():
    assert named.levenshtein("kitten", "sitting") == 3 and named.levenshtein("", "abc") == 3 and named.levenshtein("abc", "abc") == 0
    assert named.levenshtein("a" * 50, "b" * 50, limit=10) == 11


def test_detection_from_jinja_markers():
    chatml = "{% for message in messages %}{{'<|im_start|>' + message['role'] + '\\n' + message['content'] + '<|im_end|>' + '\\n'}}{% endfor %}"
    assert named.detect(chatml).name == "chatml"
    llama3 = "{% set content = '<|start_header_id|>' + message['role'] + '<|end_header_id|>\\n\\n' + message['content'] | trim + '<|eot_id|>' %}"
    assert named.detect(llama3).name == "llama3-instruct"
    assert named.detect("{{ bos_token }}{% if m['role'] == 'user' %}{{ '[INST] ' + m['content'] + ' [/INST]' }}{% endif %}").name == "mistral-instruct"
    assert named.detect("{{ '[INST] <<SYS>>\\n' + system + '\\n<</SYS>>\\n\\n' }}").name == "llama2-chat"
    assert named.detect("{{ '<start_of_turn>' + role + '\\n' + content + '<end_of_turn>\\n' }}").name == "gemma-instruct"
    assert named.detect("{{ messages | tojson }}") is None and named.detect("") is None


def test_create_from_a_bare_checkpoint_picks_the_named_template(tmp_path, monkeypatch):
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path))
    from ollama_b200.models.synth import write_synthetic_gguf
    from ollama_b200.store import manifest as M
    from ollama_b200.store.create import create_model
    from ollama_b200.store.model import get_model
    p = str(tmp_path / "m.gguf")
    jinja = "{% for message in messages %}{{'<|im_start|>' + message['role'] + '\n' + message['content'] + '<|im_end|>' + '\n'}}{% endfor %}"
    write_synthetic_gguf(p, "tiny-qwen3", "Q8_0", template=jinja)
    layer = M.new_layer(p, M.MT_MODEL)
    assert [s["status"] for s in create_model({"model": "bare", "files": {"m.gguf": layer.digest}})][-1] == "success"
    m = get_model("bare")
    assert m.template == named.named("chatml")[0] and m.options["stop"] == ["<|im_start|>", "<|im_end|>"]
    # an explicit TEMPLATE or parameter wins
    list(create_model({"model": "mine", "files": {"m.gguf": layer.digest}, "template": "{{ .Prompt }}", "parameters": {"stop": ["x"]}}))
    m = get_model("mine")
    assert m.template == "{{ .Prompt }}" and m.options["stop"] == ["x"]


REF = os.environ.get("OLLAMA_REFERENCE_DIR", "")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "template", "testdata")), reason="OLLAMA_REFERENCE_DIR does not point at a reference checkout")
def test_all_reference_goldens_and_recognised_jinja_templates():
    convs = {"user": CONV[1:2], "user-assistant-user": CONV[1:], "system-user-assistant-user": CONV}
    for l in named.LAYOUTS:
        t = Template(named.gotemplate(l))
        for case, conv in convs.items():
            with open(os.path.join(REF, "template", "testdata", l.name + ".gotmpl", case), encoding="utf-8") as f:
                assert t.execute(messages=_msgs(conv)) == f.read(), (l.name, case)
    with open(os.path.join(REF, "template", "index.json"), encoding="utf-8") as f:
        for e in json.load(f):
            got = named.detect(e["template"])
            assert got is not None and got.name == e["name"], e["name"]
