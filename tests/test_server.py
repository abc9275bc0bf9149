"""REST surface driven through the ASGI app on CPU with a tiny random-init model (pattern of the reference's
server/routes_*_test.go: handlers exercised directly, temp OLLAMA_MODELS, NDJSON streams asserted line by line)."""
import hashlib
import json
import os

import pytest


@pytest.fixture(scope="module")
def client(tmp_path_factory):
    root = tmp_path_factory.mktemp("store")
    old = {k: os.environ.get(k) for k in ("OLLAMA_MODELS", "B200_DEVICE", "OLLAMA_CONTEXT_LENGTH")}
    os.environ.update(OLLAMA_MODELS=str(root), B200_DEVICE="cpu", OLLAMA_CONTEXT_LENGTH="256")
    from starlette.testclient import TestClient

    from ollama_b200.models.synth import write_synthetic_gguf
    from ollama_b200.server.routes import create_app
    p = str(root / "m.gguf")
    write_synthetic_gguf(p, "tiny-llama", "F32")
    data = open(p, "rb").read()
    digest = "sha256:" + hashlib.sha256(data).hexdigest()
    with TestClient(create_app()) as c:
        assert c.head(f"/api/blobs/{digest}").status_code == 404
        assert c.post(f"/api/blobs/{digest}", content=data).status_code == 201
        assert c.post(f"/api/blobs/{digest}", content=data).status_code == 200
        assert c.post("/api/blobs/sha256:" + "0" * 64, content=b"x").status_code == 400
        r = c.post("/api/create", json={"model": "tiny", "files": {"m.gguf": digest}, "template": "{{ .Prompt }}",
                                        "parameters": {"temperature": 0, "num_predict": 6}, "system": "", "stream": False})
        assert r.status_code == 200 and r.json()["status"] == "success"
        yield c
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def test_root_version_tags(client):
    assert client.get("/").text == "Ollama is running"
    assert "version" in client.get("/api/version").json()
    models = client.get("/api/tags").json()["models"]
    assert models[0]["name"] == "tiny:latest" and models[0]["details"]["family"] == "llama"
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny:latest"


def test_generate_stream_and_collapse(client):
    r = client.post("/api/generate", json={"model": "tiny", "prompt": "<t300><t301><t302>", "stream": False})
    j = r.json()
    assert r.status_code == 200 and j["done"] and j["done_reason"] == "length" and j["eval_count"] == 6
    assert j["prompt_eval_count"] == 3 and j["context"][:3] == [300, 301, 302] and len(j["context"]) == 9
    assert j["response"].count("<t") == 6
    r = client.post("/api/generate", json={"model": "tiny", "prompt": "<t300><t301><t302>"})
    assert r.headers["content-type"].startswith("application/x-ndjson")
    lines = [json.loads(l) for l in r.text.strip().split("\n")]
    assert lines[-1]["done"] and not lines[0]["done"]
    assert "".join(l["response"] for l in lines) == j["response"]          # greedy: stream == collapsed
    # context continuation reuses the returned token array
    r2 = client.post("/api/generate", json={"model": "tiny", "prompt": "<t5>", "context": j["context"], "stream": False}).json()
    assert r2["context"][:9] == j["context"]


def test_generate_load_unload_and_errors(client):
    assert client.post("/api/generate", json={"model": "tiny"}).json()["done_reason"] == "load"
    assert any(m["name"] == "tiny:latest" for m in client.get("/api/ps").json()["models"])
    assert client.post("/api/generate", json={"model": "tiny", "keep_alive": 0}).json()["done_reason"] == "unload"
    assert client.get("/api/ps").json()["models"] == []
    assert client.post("/api/generate", json={"model": "missing", "prompt": "x"}).status_code == 404
    assert client.post("/api/generate", json={"prompt": "x"}).status_code == 400
    assert client.post("/api/generate", json={"model": "tiny", "prompt": "x", "options": {"top_k": "many"}}).status_code == 400
    assert client.post("/api/generate", json={"model": "tiny", "prompt": "x", "top_logprobs": 21}).status_code == 400
    assert client.post("/api/generate", json={"model": "tiny", "prompt": "x", "raw": True, "system": "s"}).status_code == 400
    assert client.post("/api/generate", content=b"{bad").status_code == 400
    r = client.post("/api/generate", json={"model": "tiny", "prompt": "<t9>", "_debug_render_only": True}).json()
    assert r["_debug_info"]["rendered_template"] == "<t9>"


def test_chat_logprobs_format(client):
    r = client.post("/api/chat", json={"model": "tiny", "messages": [{"role": "user", "content": "<t400>"}], "stream": False,
                                       "logprobs": True, "top_logprobs": 2})
    j = r.json()
    assert j["message"]["role"] == "assistant" and j["eval_count"] == 6 and len(j["logprobs"]) == 6
    assert len(j["logprobs"][0]["top_logprobs"]) == 2 and j["logprobs"][0]["logprob"] <= 0
    r = client.post("/api/generate", json={"model": "tiny", "prompt": "<t300>", "format": "json", "options": {"num_predict": 10}, "stream": False})
    text = r.json()["response"]
    assert text.strip() == "" or text.lstrip().startswith("{")             # only grammar-legal text comes out
    assert client.post("/api/generate", json={"model": "tiny", "prompt": "x", "format": "yaml"}).status_code == 400
    assert client.post("/api/chat", json={"model": "tiny", "messages": []}).json()["done_reason"] == "load"


def test_tokenize_embed_show_copy_delete(client):
    assert client.post("/api/tokenize", json={"model": "tiny", "content": "<t300>ab"}).json()["tokens"] == [300, 100, 101]
    assert client.post("/api/detokenize", json={"model": "tiny", "tokens": [300, 100, 101]}).json()["content"] == "<t300>ab"
    e = client.post("/api/embed", json={"model": "tiny", "input": ["<t500>", "<t600><t700>"]}).json()
    assert len(e["embeddings"]) == 2 and abs(sum(x * x for x in e["embeddings"][0]) - 1) < 1e-4 and e["prompt_eval_count"] == 3
    assert len(client.post("/api/embed", json={"model": "tiny", "input": "<t5>", "dimensions": 16}).json()["embeddings"][0]) == 16
    assert len(client.post("/api/embeddings", json={"model": "tiny", "prompt": "<t5>"}).json()["embedding"]) == 256
    s = client.post("/api/show", json={"model": "tiny", "verbose": True}).json()
    assert s["capabilities"] == ["completion"] and s["model_info"]["general.architecture"] == "llama"
    assert "PARAMETER temperature 0" in s["modelfile"] and any(t["name"] == "token_embd.weight" for t in s["tensors"])
    assert client.post("/api/copy", json={"source": "tiny", "destination": "copy/tiny2:v1"}).status_code == 200
    assert client.post("/api/copy", json={"source": "nope", "destination": "x"}).status_code == 404
    assert client.request("DELETE", "/api/delete", json={"model": "copy/tiny2:v1"}).status_code == 200
    assert client.request("DELETE", "/api/delete", json={"model": "copy/tiny2:v1"}).status_code == 404


def test_list_and_show_caches(client):
    srv = client.app.state.server
    a = client.post("/api/show", json={"model": "tiny"}).json()
    h0 = srv.show_cache.hits
    assert client.post("/api/show", json={"model": "tiny"}).json() == a and srv.show_cache.hits == h0 + 1
    # overlays change the answer and therefore bypass the cache
    assert client.post("/api/show", json={"model": "tiny", "system": "x"}).json()["system"] == "x" and srv.show_cache.hits == h0 + 1
    assert client.post("/api/show", json={"model": "tiny"}).json()["system"] == a["system"]
    # a changed manifest (new digest) replaces the entry
    assert client.post("/api/create", json={"model": "tiny3", "from": "tiny", "system": "one", "stream": False}).status_code == 200
    assert client.post("/api/show", json={"model": "tiny3"}).json()["system"] == "one"
    assert client.post("/api/create", json={"model": "tiny3", "from": "tiny", "system": "two", "stream": False}).status_code == 200
    assert client.post("/api/show", json={"model": "tiny3"}).json()["system"] == "two"
    t1 = client.get("/api/tags").json()["models"]
    m0 = srv.list_cache.misses
    t2 = client.get("/api/tags").json()["models"]
    assert t1 == t2 and srv.list_cache.misses == m0 and any(m["name"] == "tiny3:latest" for m in t2)
    assert client.request("DELETE", "/api/delete", json={"model": "tiny3"}).status_code == 200
    assert not any(m["name"] == "tiny3:latest" for m in client.get("/api/tags").json()["models"])


def test_builtin_renderer_and_parser_from_the_model_config(client):
    r = client.post("/api/create", json={"model": "coder", "from": "tiny", "renderer": "qwen3-coder", "parser": "qwen3-coder", "stream": False})
    assert r.status_code == 200
    s = client.post("/api/show", json={"model": "coder"}).json()
    assert s["renderer"] == "qwen3-coder" and s["parser"] == "qwen3-coder" and "tools" in s["capabilities"]
    assert "RENDERER qwen3-coder" in s["modelfile"] and "PARSER qwen3-coder" in s["modelfile"]
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {"x": {"type": "integer"}}}}}]
    d = client.post("/api/chat", json={"model": "coder", "messages": [{"role": "user", "content": "hi"}], "tools": tools,
                                       "_debug_render_only": True}).json()
    p = d["_debug_info"]["rendered_template"]
    assert p.startswith("<|im_start|>system\nYou are Qwen") and "<function>\n<name>f</name>" in p and p.endswith("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n")
    # the request still runs end to end with the built-in parser in the stream
    j = client.post("/api/chat", json={"model": "coder", "messages": [{"role": "user", "content": "<t400>"}], "tools": tools, "stream": False,
                                       "options": {"num_predict": 4}}).json()
    assert j["done"] and j["eval_count"] == 4 and "content" in j["message"]


def test_tool_calls_of_the_builtin_parser_carry_ids_and_indices_and_roles_compare_in_lower_case(client, monkeypatch):
    """A scripted model output through /api/chat: each parsed call gets an id and its running index (api/types_test.go:408-430 of the
    reference: the index is always present); an upper-case role is the same as its lower-case form (api/types_test.go:286-307)."""
    from ollama_b200.engine.runner import CompletionChunk, Runner
    script = ["Let me look.", "<tool_call>\n<function=f>\n<parameter=x>\n3\n</parameter>\n</function>\n</tool_call>",
              "<tool_call>\n<function=f>\n<parameter=x>\n4\n</parameter>\n</function>\n</tool_call>"]

    def scripted(self, req):
        for i, piece in enumerate(script):
            yield CompletionChunk(content=piece)
        yield CompletionChunk(done=True, done_reason="stop", eval_count=len(script))

    monkeypatch.setattr(Runner, "completion", scripted)
    assert client.post("/api/create", json={"model": "coder2", "from": "tiny", "renderer": "qwen3-coder", "parser": "qwen3-coder", "stream": False}).status_code == 200
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {"x": {"type": "integer"}}}}}]
    j = client.post("/api/chat", json={"model": "coder2", "messages": [{"role": "USER", "content": "hi"}], "tools": tools, "stream": False}).json()
    calls = j["message"]["tool_calls"]
    assert [c["function"]["index"] for c in calls] == [0, 1] and [c["function"]["arguments"] for c in calls] == [{"x": 3}, {"x": 4}]
    assert all(c["id"].startswith("call_") for c in calls) and calls[0]["id"] != calls[1]["id"] and j["message"]["content"] == "Let me look."
    d = client.post("/api/chat", json={"model": "coder2", "messages": [{"role": "SYSTEM", "content": "be kind"}, {"role": "User", "content": "hi"}],
                                       "_debug_render_only": True}).json()["_debug_info"]["rendered_template"]
    assert d.startswith("<|im_start|>system\nbe kind<|im_end|>\n<|im_start|>user\nhi<|im_end|>")


def test_metrics_route_reports_runner_totals(client):
    client.post("/api/generate", json={"model": "tiny", "prompt": "<t400><t401>", "stream": False, "options": {"num_predict": 3}})
    r = client.get("/metrics")
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
    vals: dict[str, float] = {}
    for line in r.text.splitlines():
        if line and not line.startswith("#"):
            k, v = line.rsplit(" ", 1)
            k = k.split("{")[0] + ("{reason=" + k.split('reason="')[1] if 'reason="' in k else "")     # runners are shared by models of one blob
            vals[k] = vals.get(k, 0.0) + float(v)
    assert vals["ollama_b200_loaded_models"] >= 1, r.text
    assert vals["ollama_b200_requests_total"] >= 1 and vals["ollama_b200_generated_tokens_total"] >= 3
    assert vals["ollama_b200_ttft_seconds_total"] > 0 and vals["ollama_b200_decode_steps_total"] >= 2
    assert vals['ollama_b200_done_total{reason=length"}'] >= 1
    assert "# TYPE ollama_b200_requests_total counter" in r.text


def test_draft_model_from_create_reaches_the_runner(client):
    """``draft_files`` (Modelfile DRAFT) becomes a draft layer; the scheduler hands it to the runner, which then speculates."""
    import glob
    tiny = client.post("/api/show", json={"model": "tiny"}).json()
    ggufs = [p for p in glob.glob(os.path.join(os.environ["OLLAMA_MODELS"], "blobs", "sha256-*")) if open(p, "rb").read(4) == b"GGUF"]
    digest = "sha256:" + os.path.basename(ggufs[0])[len("sha256-"):]
    r = client.post("/api/create", json={"model": "spec", "from": "tiny", "draft_files": {"draft.gguf": digest}, "parameters": {"num_ctx": 192},
                                         "stream": False})
    assert r.status_code == 200 and tiny["details"]["format"] == "gguf"
    a = client.post("/api/generate", json={"model": "tiny", "prompt": "<t400><t401>", "stream": False, "options": {"num_predict": 12, "num_ctx": 192}}).json()
    b = client.post("/api/generate", json={"model": "spec", "prompt": "<t400><t401>", "stream": False, "options": {"num_predict": 12}}).json()
    assert a["response"] == b["response"] and b["eval_count"] == 12
    text = client.get("/metrics").text
    accepted = [float(l.rsplit(" ", 1)[1]) for l in text.splitlines() if l.startswith("ollama_b200_draft_accepted_tokens_total")]
    assert accepted and max(accepted) > 0


def test_create_from_existing_model(client):
    r = client.post("/api/create", json={"model": "child", "from": "tiny", "system": "be brief", "parameters": {"stop": ["<t1>"]},
                                         "stream": False})
    assert r.status_code == 200
    s = client.post("/api/show", json={"model": "child"}).json()
    assert s["system"] == "be brief" and "stop" in s["parameters"] and "temperature" in s["parameters"]
    assert client.post("/api/create", json={"model": "x", "from": "nope", "stream": False}).status_code == 404
    assert client.post("/api/create", json={"model": "x", "stream": False}).status_code == 400


def test_openai_and_anthropic_facades(client):
    body = {"model": "tiny", "messages": [{"role": "user", "content": [{"type": "text", "text": "<t400>"}]}], "max_tokens": 4}
    j = client.post("/v1/chat/completions", json=body).json()
    assert j["object"] == "chat.completion" and j["choices"][0]["finish_reason"] == "length" and j["usage"]["completion_tokens"] == 4
    r = client.post("/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}})
    events = [l[6:] for l in r.text.split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]" and json.loads(events[-2])["usage"]["completion_tokens"] == 4
    assert json.loads(events[0])["choices"][0]["delta"]["role"] == "assistant"
    j = client.post("/v1/completions", json={"model": "tiny", "prompt": "<t400>", "max_tokens": 3}).json()
    assert j["object"] == "text_completion" and j["choices"][0]["text"].count("<t") == 3
    j = client.post("/v1/embeddings", json={"model": "tiny", "input": ["<t5>"]}).json()
    assert j["data"][0]["object"] == "embedding" and len(j["data"][0]["embedding"]) == 256
    assert client.post("/v1/chat/completions", json={"model": "nope", "messages": [{"role": "user", "content": "x"}]}).status_code == 404
    assert client.get("/v1/models/tiny").json()["id"] == "tiny:latest"
    j = client.post("/v1/responses", json={"model": "tiny", "input": "<t400>", "max_output_tokens": 3}).json()
    assert j["status"] == "completed" and j["usage"]["output_tokens"] == 3
    j = client.post("/v1/messages", json={"model": "tiny", "messages": [{"role": "user", "content": "<t400>"}], "max_tokens": 3}).json()
    assert j["type"] == "message" and j["stop_reason"] == "max_tokens" and j["usage"]["output_tokens"] == 3
    r = client.post("/v1/messages", json={"model": "tiny", "messages": [{"role": "user", "content": "<t400>"}], "max_tokens": 3, "stream": True})
    assert "event: message_start" in r.text and "event: message_stop" in r.text


def test_openai_stream_frames_and_message_conversion_follow_the_reference_cases():
    """The wire cases of middleware/openai_test.go:92-812 and :926-1220 of the reference on the two pure converters."""
    from ollama_b200.server.openai import ChatStreamState, _messages, _options, chat_stream_frames
    base = {"id": "chatcmpl-test", "object": "chat.completion.chunk", "created": 1, "model": "m", "system_fingerprint": "fp_ollama"}

    def run(objs, usage=False):
        st, out = ChatStreamState(), []
        for o in objs:
            out += chat_stream_frames(st, o, base, usage)
        return out

    # reasoning and answer in one response: two chunks, then the finish chunk with an empty delta, then usage with no choices
    f = run([{"message": {"thinking": "reasoning", "content": "final answer"}, "done": True, "done_reason": "stop", "prompt_eval_count": 3, "eval_count": 2}], True)
    assert len(f) == 4 and f[0]["choices"][0]["delta"] == {"role": "assistant", "reasoning": "reasoning"} and f[0]["choices"][0]["finish_reason"] is None
    assert f[1]["choices"][0]["delta"] == {"content": "final answer"} and f[2]["choices"][0] == {"index": 0, "delta": {}, "finish_reason": "stop"}
    assert f[3]["choices"] == [] and f[3]["usage"]["total_tokens"] == 5
    # reasoning with a call, not final: two chunks and nothing else
    call = {"id": "call_234", "function": {"index": 0, "name": "get_weather", "arguments": {"location": "Portland"}}}
    f = run([{"message": {"thinking": "reasoning", "tool_calls": [call]}, "done": False}])
    assert len(f) == 2 and "tool_calls" not in f[0]["choices"][0]["delta"] and f[1]["choices"][0]["delta"]["tool_calls"][0]["function"]["name"] == "get_weather"
    assert f[1]["choices"][0]["delta"]["tool_calls"][0]["function"]["arguments"] == '{"location": "Portland"}'
    # the role is on the first chunk only; the finish chunk closes the stream
    f = run([{"message": {"content": "Hello"}}, {"message": {"content": " world"}}, {"message": {"content": "!"}, "done": True, "done_reason": "stop"}])
    assert [c["choices"][0]["delta"] for c in f] == [{"role": "assistant", "content": "Hello"}, {"content": " world"}, {"content": "!"}, {}]
    assert all(c["created"] == 1 for c in f)
    # the closing response with an empty message adds no empty content chunk; its finish reason passes through
    f = run([{"message": {"content": "Hi"}}, {"message": {"content": ""}, "done": True, "done_reason": "length", "prompt_eval_count": 3, "eval_count": 1}], True)
    assert len(f) == 3 and f[1]["choices"][0] == {"index": 0, "delta": {}, "finish_reason": "length"} and f[2]["choices"] == []
    # ... unless it carries the log-probabilities of the last token
    f = run([{"message": {"content": "Hi"}}, {"message": {"content": ""}, "done": True, "done_reason": "stop", "logprobs": [{"token": "Hi", "logprob": -0.1}]}])
    assert len(f) == 3 and f[1]["choices"][0]["logprobs"]["content"][0]["logprob"] == -0.1 and f[2]["choices"][0]["delta"] == {}
    # an empty completion still opens with the role; a streamed call turns "stop" into "tool_calls" but leaves "length" alone
    f = run([{"message": {"content": ""}, "done": True, "done_reason": "stop"}])
    assert len(f) == 2 and f[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""} and f[1]["choices"][0]["finish_reason"] == "stop"
    assert run([{"message": {"tool_calls": [call]}}, {"message": {}, "done": True, "done_reason": "stop"}])[-1]["choices"][0]["finish_reason"] == "tool_calls"
    assert run([{"message": {"tool_calls": [call]}}, {"message": {}, "done": True, "done_reason": "length"}])[-1]["choices"][0]["finish_reason"] == "length"

    args = '{"location": "Paris, France", "format": "celsius"}'
    calls = [{"id": "id_abc", "type": "function", "function": {"name": "get_current_weather", "arguments": args}}]
    m = _messages({"messages": [{"role": "user", "content": "weather?"}, {"role": "assistant", "reasoning": "let me see", "tool_calls": calls},
                                {"role": "tool", "tool_call_id": "id_abc", "content": "20 degrees"}, {"role": "tool", "name": "other", "content": "x"},
                                {"role": "developer", "content": "rules"}]})
    assert m[1] == {"role": "assistant", "content": "", "thinking": "let me see",
                    "tool_calls": [{"id": "id_abc", "function": {"name": "get_current_weather", "arguments": {"location": "Paris, France", "format": "celsius"}}}]}
    assert m[2]["tool_name"] == "get_current_weather" and m[2]["tool_call_id"] == "id_abc" and m[3]["tool_name"] == "other" and m[4]["role"] == "system"
    o = _options({"max_tokens": 999, "seed": 123, "stop": ["\n", "stop"], "temperature": 3.0, "frequency_penalty": 4.0, "presence_penalty": 5.0, "top_p": 6.0})
    assert o == {"num_predict": 999, "seed": 123, "stop": ["\n", "stop"], "temperature": 3.0, "frequency_penalty": 4.0, "presence_penalty": 5.0, "top_p": 6.0}
    assert _options({}) == {"temperature": 1.0, "top_p": 1.0} and _options({"stop": "x"})["stop"] == ["x"]


def test_chat_prompt_truncation_on_the_reference_cases():
    """Text cases of server/prompt_test.go:24-320 of the reference: what is kept when the conversation does not fit, system messages
    that survive, no truncation on request, and how many tokenisations that costs."""
    from ollama_b200.server.prompt import chat_prompt
    from ollama_b200.text.template import Template
    t = Template("{{- if .System }}{{ .System }} {{ end }}\n{{- if .Prompt }}{{ .Prompt }} {{ end }}\n{{- if .Response }}{{ .Response }} {{ end }}")
    render = lambda ms: t.execute(messages=ms)                  # noqa: E731
    n_calls = [0]

    def count(s):
        n_calls[0] += 1
        return len(s.split())

    harry = [{"role": "user", "content": "You're a test, Harry!"}, {"role": "assistant", "content": "I-I'm a what?"},
             {"role": "user", "content": "A test. And a thumping good one at that, I'd wager."}]
    whole = "You're a test, Harry! I-I'm a what? A test. And a thumping good one at that, I'd wager. "
    assert chat_prompt(render, count, harry, 64)[0] == whole
    assert chat_prompt(render, count, harry, 1)[0] == "A test. And a thumping good one at that, I'd wager. "
    assert chat_prompt(render, count, harry, 10, truncate=False)[0] == whole
    system = {"role": "system", "content": "You are the Test Who Lived."}
    assert chat_prompt(render, count, [system] + harry, 2048)[0] == "You are the Test Who Lived. " + whole
    assert chat_prompt(render, count, harry[:2] + [system] + harry[2:], 2048)[0] == \
        "You're a test, Harry! I-I'm a what? You are the Test Who Lived. A test. And a thumping good one at that, I'd wager. "
    p, used = chat_prompt(render, count, [system] + harry, 18)          # the system message survives the cut
    assert p == "You are the Test Who Lived. A test. And a thumping good one at that, I'd wager. " and [m["role"] for m in used] == ["system", "user"]
    five = [{"role": "user" if i % 2 == 0 else "assistant", "content": f"message {i}"} for i in range(5)]
    n_calls[0] = 0
    chat_prompt(render, count, five, 2048)
    assert n_calls[0] == 1                                              # a chat that fits is tokenised once
    n_calls[0] = 0
    assert chat_prompt(render, count, five, 2)[0] == "message 4 " and n_calls[0] <= 5
    assert chat_prompt(render, count, [], 10)[0] == ""


def test_host_allow_list_and_cors(client):
    assert client.get("/", headers={"Host": "evil.example.com"}).status_code == 403
    assert client.get("/", headers={"Host": "localhost:11434"}).status_code == 200
    r = client.options("/api/generate", headers={"Origin": "http://localhost:3000", "Access-Control-Request-Method": "POST"})
    assert r.headers.get("access-control-allow-origin") == "http://localhost:3000"
    r = client.options("/api/generate", headers={"Origin": "http://evil.example.com", "Access-Control-Request-Method": "POST"})
    assert "access-control-allow-origin" not in r.headers


def test_malformed_request_fields_are_client_errors(client):
    """Every route answers a body whose fields have the wrong JSON kind with a 4xx (or a normal answer), never a 5xx:
    the native routes check the kinds up front, the OpenAI and Anthropic façades check theirs before translating."""
    import random
    rnd = random.Random(11)
    junk = [None, True, 0, -1, 1.5, "x", "", [], {}, [1, "a"], {"a": 1}, "tiny", [{"role": "user", "content": "hi"}], [{"role": 1, "content": [1]}],
            {"type": "object"}, "json", 1e30, [[]], {"num_predict": 2}, {"num_predict": "x"}, [{"type": "function", "function": {"name": "f"}}],
            [{"function": 1}], "5m", -5]
    keys = {"/api/generate": ["model", "prompt", "suffix", "system", "template", "context", "stream", "raw", "format", "options", "keep_alive", "think", "images", "logprobs", "top_logprobs"],
            "/api/chat": ["model", "messages", "tools", "stream", "format", "options", "keep_alive", "think", "logprobs", "top_logprobs"],
            "/api/embed": ["model", "input", "truncate", "options", "dimensions", "keep_alive"], "/api/embeddings": ["model", "prompt", "options"],
            "/api/show": ["model", "verbose", "system", "options"], "/api/tokenize": ["model", "content", "add_special"], "/api/detokenize": ["model", "tokens"],
            "/api/create": ["model", "from", "files", "adapters", "template", "system", "parameters", "messages", "quantize", "stream", "draft_files", "license"],
            "/api/copy": ["source", "destination"],
            "/v1/chat/completions": ["model", "messages", "tools", "stream", "max_tokens", "temperature", "response_format", "stop", "logprobs", "top_logprobs", "stream_options", "reasoning_effort", "seed"],
            "/v1/completions": ["model", "prompt", "max_tokens", "stream", "suffix", "stop"], "/v1/embeddings": ["model", "input", "encoding_format", "dimensions"],
            "/v1/responses": ["model", "input", "instructions", "tools", "stream", "max_output_tokens"],
            "/v1/messages": ["model", "messages", "max_tokens", "system", "tools", "stream", "thinking", "stop_sequences"]}
    seen = set()
    for _ in range(260):
        path = rnd.choice(list(keys))
        body = {k: rnd.choice(junk) for k in rnd.sample(keys[path], rnd.randint(0, len(keys[path])))}
        if rnd.random() < 0.7:
            body["model"] = "tiny"
        if "stream" in keys[path]:
            body["stream"] = False
        if path == "/api/create":
            body["model"] = rnd.choice(["t2", "", "a/b:c"])
        r = client.post(path, json=body)
        seen.add(r.status_code)
        assert r.status_code < 500 or r.status_code in (501, 503), (path, body, r.status_code, r.text[:200])
    assert 400 in seen and 200 in seen
    assert client.post("/api/chat", json={"model": "tiny", "messages": "hi"}).json()["error"] == "invalid request: 'messages' must be an array of objects"
    assert client.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "x"}], "temperature": "hot"}).status_code == 400


def test_image_input_is_refused_not_dropped(client):
    """server/routes.go (images add the vision capability to a request): a text model answers 400; so does this engine for any
    model, since it has no vision tower - the images are never silently left out of the prompt."""
    r = client.post("/api/chat", json={"model": "tiny", "messages": [{"role": "user", "content": "what is this?", "images": ["aGk="]}], "stream": False})
    assert r.status_code == 400 and "does not support vision" in r.json()["error"]
    r = client.post("/api/generate", json={"model": "tiny", "prompt": "describe", "images": ["aGk="], "stream": False})
    assert r.status_code == 400 and "does not support vision" in r.json()["error"]
    r = client.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": [
        {"type": "text", "text": "hi"}, {"type": "image_url", "image_url": {"url": "data:image/png;base64,aGk="}}]}]})
    assert r.status_code == 400
    r = client.post("/api/chat", json={"model": "tiny", "messages": [{"role": "user", "content": "<t300>"}], "stream": False})
    assert r.status_code == 200


def test_inference_model_cache_and_recommendations(client, tmp_path, monkeypatch):
    """server/model_inference_cache_test.go: one load per manifest digest, a private copy per request, a new digest reloads;
    server/model_recommendations_test.go: defaults, snapshot, stale-while-revalidate, back-off, nothing fetched with cloud off."""
    from ollama_b200.server import caches as C
    loads = []

    def load(name):
        from ollama_b200.store.model import get_model
        loads.append(name)
        return get_model(name)

    c = C.InferenceModelCache(load)
    a, b = c.get("tiny"), c.get("tiny:latest")
    assert loads == ["tiny"] and a is not b and a.digest == b.digest and c.hits == 1
    a.options["temperature"] = 9
    a.adapter_paths.append("x")
    assert "x" not in c.get("tiny").adapter_paths and c.get("tiny").options.get("temperature") != 9
    assert a.capabilities() == b.capabilities() and a._kv is b._kv
    r = client.post("/api/create", json={"model": "tiny", "from": "tiny", "system": "changed", "stream": False})
    assert r.status_code == 200
    assert c.get("tiny").system == "changed" and len(loads) == 2          # the manifest digest moved: loaded again
    import pytest
    from ollama_b200.store.model import ModelNotFound
    with pytest.raises(ModelNotFound):
        c.get("absent")
    r = client.post("/api/create", json={"model": "tiny", "from": "tiny", "system": "", "stream": False})
    assert r.status_code == 200

    # recommendations
    assert client.get("/api/experimental/model-recommendations").json()["recommendations"][0]["model"]
    clock = [0.0]
    answers = [[{"model": "m1", "description": "d", "vram_bytes": 5}], RuntimeError("down"), RuntimeError("down"), [{"model": "m2", "description": ""}]]

    def fetch():
        v = answers.pop(0)
        if isinstance(v, Exception):
            raise v
        return v

    monkeypatch.delenv("OLLAMA_NO_CLOUD", raising=False)
    snap = str(tmp_path / "rec.json")
    rc = C.RecommendationsCache(fetch, snap, now=lambda: clock[0])
    assert rc.source == "default" and rc.get_swr(background=False)[0]["model"] == C.DEFAULT_RECOMMENDATIONS[0]["model"]   # stale first ...
    assert rc.get()[0] == {"model": "m1", "description": "d", "vram_bytes": 5} and rc.source == "remote"              # ... fresh after
    assert C.RecommendationsCache(fetch, snap).source == "snapshot"
    rc.get_swr(background=False)
    assert len(answers) == 3                                               # inside the 4 h refresh interval: no fetch
    clock[0] += 4 * 3600 + 1
    rc.get_swr(background=False)
    assert rc.failures == 1 and rc.get()[0]["model"] == "m1"               # failure keeps the list
    clock[0] += 299
    rc.get_swr(background=False)
    assert len(answers) == 2                                               # first back-off step: 5 minutes
    clock[0] += 2
    rc.get_swr(background=False)
    assert rc.failures == 2
    clock[0] += 901
    rc.get_swr(background=False)
    assert rc.failures == 0 and rc.get()[0]["model"] == "m2"
    monkeypatch.setenv("OLLAMA_NO_CLOUD", "1")
    quiet = C.RecommendationsCache(lambda: (_ for _ in ()).throw(AssertionError("fetched")), str(tmp_path / "none.json"))
    quiet.get_swr(background=False)
    assert quiet.source == "default" and quiet.failures == 0
    for bad in (None, [], [{"description": "x"}], [{"model": "m", "vram_bytes": "big"}], [{"model": "m", "context_length": -1}]):
        with pytest.raises(ValueError):
            C.validate_recommendations(bad)


def test_anthropic_web_search_server_tool_loop(client):
    """middleware/anthropic_test.go (web search): calls of the built-in tool are answered by the server, results go back to the
    model, at most three searches, every search shows up as a server_tool_use + web_search_tool_result pair."""
    from ollama_b200.server import anthropic as A
    tools, wants = A.split_server_tools([{"type": "web_search_20250305", "name": "web_search"}, {"name": "web_search", "input_schema": {}},
                                         {"name": "calc", "description": "adds", "input_schema": {"type": "object"}}])
    assert wants and [t["function"]["name"] for t in tools] == ["web_search", "calc"] and tools[0] is A.WEB_SEARCH_TOOL
    assert A.split_server_tools([{"name": "web_search", "input_schema": {}}]) == ([{"type": "function", "function": {"name": "web_search", "description": "", "parameters": {}}}], False)

    def call(q):
        return {"message": {"role": "assistant", "content": "", "tool_calls": [{"id": "c1", "function": {"name": "web_search", "arguments": {"query": q}}}]},
                "prompt_eval_count": 10, "eval_count": 5, "done_reason": "stop"}

    answer = {"message": {"role": "assistant", "content": "It is sunny."}, "prompt_eval_count": 30, "eval_count": 7, "done_reason": "stop"}
    native = {"model": "m", "messages": [{"role": "user", "content": "weather?"}], "tools": [A.WEB_SEARCH_TOOL], "options": {}}
    seen = []

    def chat_once(req):
        seen.append(req["messages"])
        return answer

    found = [{"title": "Weather", "url": "https://w.example", "content": "sunny"}]
    out = A.run_web_search_loop(chat_once, native, call("weather today"), lambda q, n: found, "msg_abc", "m")
    assert [b["type"] for b in out["content"]] == ["server_tool_use", "web_search_tool_result", "text"]
    assert out["content"][0] == {"type": "server_tool_use", "id": "srvtoolu_abc", "name": "web_search", "input": {"query": "weather today"}}
    assert out["content"][1]["content"] == [{"type": "web_search_result", "url": "https://w.example", "title": "Weather"}]
    assert out["usage"] == {"input_tokens": 40, "output_tokens": 12} and out["stop_reason"] == "end_turn"
    assert seen[0][-1] == {"role": "tool", "content": "Title: Weather\nURL: https://w.example\nContent: sunny\n\n", "tool_call_id": "c1"}
    assert seen[0][-2]["tool_calls"][0]["function"]["arguments"] == {"query": "weather today"} and len(native["messages"]) == 1
    # a model that keeps searching is stopped after three searches
    n = [0]

    def chat_again(req):
        n[0] += 1
        return call(f"again {n[0]}")

    out = A.run_web_search_loop(chat_again, native, call("q0"), lambda q, k: found, "msg_x", "m")
    assert n[0] == 3 and [b["id"] for b in out["content"] if b["type"] == "server_tool_use"] == ["srvtoolu_x", "srvtoolu_x_2", "srvtoolu_x_3", "srvtoolu_x_4"]
    assert out["content"][-1]["content"] == {"type": "web_search_tool_result_error", "error_code": "max_uses_exceeded"}
    # failures of the search, of the follow-up turn and an empty query are results with an error code, not exceptions

    def down(q, k):
        raise OSError("no route")

    assert A.run_web_search_loop(chat_once, native, call("q"), down, "msg_y", "m")["content"][1]["content"]["error_code"] == "unavailable"
    assert A.run_web_search_loop(chat_once, native, call("  "), lambda q, k: found, "msg_y", "m")["content"][1]["content"]["error_code"] == "invalid_request"

    def broken(req):
        raise RuntimeError("runner died")

    assert A.run_web_search_loop(broken, native, call("q"), lambda q, k: found, "msg_y", "m")["content"][-1]["content"]["error_code"] == "api_error"
    # the finished message as a stream
    names = [name for name, _ in A.message_events(A.run_web_search_loop(chat_once, native, call("q"), lambda q, k: found, "msg_z", "m"))]
    assert names == ["message_start", "content_block_start", "content_block_delta", "content_block_stop", "content_block_start", "content_block_stop",
                     "content_block_start", "content_block_delta", "content_block_stop", "message_delta", "message_stop"]
    # through the route: a model without tool support refuses, as it does for client tools
    r = client.post("/v1/messages", json={"model": "tiny", "max_tokens": 4, "messages": [{"role": "user", "content": "hi"}],
                                         "tools": [{"type": "web_search_20250305", "name": "web_search"}]})
    assert r.status_code == 400 and "does not support tools" in r.json()["error"]["message"]


def test_openai_transcription_route_parses_the_upload_and_refuses_what_the_model_cannot_hear(client):
    """middleware/openai.go:1274-1340: multipart form with model and file; the audio travels as media of a chat request, which a
    text model refuses."""
    r = client.post("/v1/audio/transcriptions", data={"model": "tiny"})
    assert r.status_code == 400 and "file is required" in r.json()["error"]["message"]
    r = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", b"RIFF....", "audio/wav")})
    assert r.status_code == 400 and "model is required" in r.json()["error"]["message"]
    r = client.post("/v1/audio/transcriptions", data={"model": "tiny"}, files={"file": ("a.wav", b"", "audio/wav")})
    assert r.status_code == 400 and "empty" in r.json()["error"]["message"]
    r = client.post("/v1/audio/transcriptions", data={"model": "tiny", "language": "en"}, files={"file": ("a.wav", b"RIFF1234", "audio/wav")})
    assert r.status_code == 400 and "does not support vision" in r.json()["error"]["message"]
    r = client.post("/v1/audio/transcriptions", data={"model": "absent"}, files={"file": ("a.wav", b"RIFF1234", "audio/wav")})
    assert r.status_code == 404
