"""Model names, Modelfile parsing, manifests/blobs, create + quantize, env config and option handling."""
import math
import os

import pytest

from ollama_b200 import envconfig
from ollama_b200.api.types import OptionError, default_options, format_parameters, options_from_map, parse_keep_alive, parse_think
from ollama_b200.store import manifest as M
from ollama_b200.store.modelfile import ModelfileError, parse_modelfile
from ollama_b200.store.names import parse_name


def test_names():
    n = parse_name("llama3")
    assert str(n) == "registry.ollama.ai/library/llama3:latest" and n.display() == "llama3:latest" and n.valid
    n = parse_name("example.com:5000/ns/model:7b-q4_K_M")
    assert (n.host, n.namespace, n.model, n.tag) == ("example.com:5000", "ns", "model", "7b-q4_K_M") and n.display() == str(n)
    assert parse_name("user/m").display() == "user/m:latest" and parse_name("https://h.io/a/b:c").host == "h.io"
    assert n.filepath() == "example.com:5000/ns/model/7b-q4_K_M"
    for bad in ("", "a b", "x/y/z/w/v:::", "-bad", "m:ta g"):
        assert not parse_name(bad).valid


def test_modelfile_parser():
    mf = parse_modelfile('# comment\nFROM llama3\nPARAMETER temperature 0.5\nparameter stop "<|a|>"\nPARAMETER stop b\n'
                         'SYSTEM """multi\nline"""\nMESSAGE user hello there\nTEMPLATE "{{ .Prompt }}"\nLICENSE MIT\nADAPTER ./lora.gguf\n')
    req = mf.create_request()
    assert req["from"] == "llama3" and req["system"] == "multi\nline" and req["template"] == "{{ .Prompt }}"
    assert req["parameters"] == {"temperature": 0.5, "stop": ["<|a|>", "b"]} and req["messages"] == [{"role": "user", "content": "hello there"}]
    assert req["license"] == ["MIT"] and req["adapter_paths"] == ["./lora.gguf"]
    again = parse_modelfile(str(mf)).create_request()          # serialise -> parse is stable
    assert again == req
    with pytest.raises(ModelfileError, match="no FROM line"):
        parse_modelfile("SYSTEM hi\n")
    with pytest.raises(ModelfileError, match="command must be one of"):
        parse_modelfile("FROM x\nBOGUS y\n")
    with pytest.raises(ModelfileError, match="role"):
        parse_modelfile("FROM x\nMESSAGE robot hi\n")
    with pytest.raises(OptionError):
        parse_modelfile("FROM x\nPARAMETER temperature hot\n").create_request()
    with pytest.raises(OptionError, match="unknown parameter"):
        parse_modelfile("FROM x\nPARAMETER nope 1\n").create_request()
    assert parse_modelfile("FROM x\nPARAMETER mirostat 1\n").create_request().get("parameters") in (None, {})   # deprecated: ignored


def test_manifest_blob_store(tmp_path, monkeypatch):
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path))
    a = M.new_layer(b"hello", M.MT_SYSTEM)
    b = M.new_layer(b"hello", M.MT_SYSTEM)
    assert a.digest == b.digest == "sha256:2cf24dba5fb0a30e26e83b2ac5b9e29e1b161e5c1fa7425e73043362938b9824" and a.size == 5
    assert os.path.basename(a.path()) == "sha256-" + a.digest[7:]
    cfg = M.new_layer(b"{}", M.MT_CONFIG)
    n = parse_name("me/thing:v1")
    M.write_manifest(n, cfg, [a])
    assert os.path.exists(tmp_path / "manifests" / "registry.ollama.ai" / "me" / "thing" / "v1")
    m = M.read_manifest(n)
    assert m.layers[0].digest == a.digest and m.size() == 7 and m.layer(M.MT_SYSTEM).read() == b"hello"
    M.copy_model(n, parse_name("me/other"))
    assert sorted(x.display() for x, _ in M.list_manifests()) == ["me/other:latest", "me/thing:v1"]
    orphan = M.new_layer(b"orphan", M.MT_LICENSE)
    M.delete_model(n)
    assert not os.path.exists(orphan.path()) and os.path.exists(a.path())          # still referenced by me/other
    M.delete_model(parse_name("me/other"))
    assert not os.path.exists(a.path())
    with pytest.raises(M.StoreError):
        M.blob_path("sha256:xyz")
    with pytest.raises(M.StoreError):
        M.read_manifest(n)


def test_create_with_quantize(tmp_path, monkeypatch):
    monkeypatch.setenv("OLLAMA_MODELS", str(tmp_path))
    from ollama_b200.gguf.reader import open_gguf
    from ollama_b200.gguf.types import GGMLType
    from ollama_b200.models.synth import write_synthetic_gguf
    from ollama_b200.store.create import CreateError, create_model
    from ollama_b200.store.model import get_model
    p = str(tmp_path / "f16.gguf")
    write_synthetic_gguf(p, "tiny-qwen3", "F16")
    layer = M.new_layer(p, M.MT_MODEL)
    status = [s["status"] for s in create_model({"model": "q", "files": {"f16.gguf": layer.digest}, "quantize": "q4_K_M"})]
    assert status[-1] == "success" and any("quantizing" in s for s in status)
    m = get_model("q")
    assert m.config["file_type"] == "Q4_K_M" and m.config["model_family"] == "qwen3"
    g = open_gguf(m.model_path)
    assert g.tensors["output.weight"].dtype == GGMLType.Q6_K and g.tensors["blk.1.attn_q.weight"].dtype == GGMLType.Q4_K
    assert g.tensors["blk.0.attn_norm.weight"].dtype == GGMLType.F32 and g.tensors["blk.1.ffn_down.weight"].dtype == GGMLType.Q6_K
    g.close()
    with pytest.raises(CreateError, match="only supported for F16 and F32"):
        list(create_model({"model": "q2", "from": "q", "quantize": "q8_0"}))
    with pytest.raises(CreateError, match="unsupported quantization"):
        list(create_model({"model": "q3", "files": {"f16.gguf": layer.digest}, "quantize": "q3_k_s"}))


def test_envconfig(monkeypatch):
    for k in ("OLLAMA_HOST", "OLLAMA_KEEP_ALIVE", "OLLAMA_ORIGINS", "OLLAMA_DEBUG", "OLLAMA_NUM_PARALLEL"):
        monkeypatch.delenv(k, raising=False)
    assert str(envconfig.host()) == "http://127.0.0.1:11434" and envconfig.keep_alive() == 300 and envconfig.num_parallel() == 1
    cases = {"1.2.3.4": "http://1.2.3.4:11434", ":1234": "http://127.0.0.1:1234", "example.com:99": "http://example.com:99",
             "https://example.com": "https://example.com:443", "http://h/path": "http://h:80/path", "[::1]": "http://[::1]:11434",
             "[::1]:8080": "http://[::1]:8080", "0.0.0.0:66000": "http://0.0.0.0:11434", "ollama.com": "https://ollama.com:443"}
    for k, v in cases.items():
        monkeypatch.setenv("OLLAMA_HOST", k)
        assert str(envconfig.host()) == v, k
    for k, v in {"5m": 300, "1h30m": 5400, "42": 42, "-1": math.inf, "-1s": math.inf, "0": 0, "junk": 300}.items():
        monkeypatch.setenv("OLLAMA_KEEP_ALIVE", k)
        assert envconfig.keep_alive() == v, k
    monkeypatch.setenv("OLLAMA_ORIGINS", "http://a.com,https://b.io")
    o = envconfig.allowed_origins()
    assert o[:2] == ["http://a.com", "https://b.io"] and "http://localhost:*" in o and "app://*" in o
    monkeypatch.setenv("OLLAMA_DEBUG", "2")
    assert envconfig.log_level() == 5
    monkeypatch.setenv("OLLAMA_NUM_PARALLEL", "x")
    assert envconfig.num_parallel() == 1 and "OLLAMA_MAX_QUEUE" in envconfig.as_map()


def test_options_and_wire_values():
    o = default_options()
    assert o["temperature"] == 0.8 and o["top_k"] == 40 and o["num_predict"] == -1 and o["num_keep"] == 4 and o["seed"] == -1
    options_from_map(o, {"temperature": 0, "top_k": 5.0, "stop": "x", "use_mmap": True, "unknown": 1, "seed": None})
    assert o["temperature"] == 0.0 and o["top_k"] == 5 and o["stop"] == ["x"] and o["use_mmap"] is True and "unknown" not in o
    for bad in ({"top_k": "5"}, {"temperature": "hot"}, {"use_mmap": 1}, {"stop": [1]}, {"num_ctx": True}):
        with pytest.raises(OptionError):
            options_from_map(default_options(), bad)
    assert parse_keep_alive("10m") == 600 and parse_keep_alive(-1) == math.inf and parse_keep_alive(0) == 0 and parse_keep_alive(None) is None
    assert parse_keep_alive("30") == 30
    with pytest.raises(ValueError):
        parse_keep_alive("soon")
    assert parse_think(True) is True and parse_think("high") == "high" and parse_think(None) is None
    with pytest.raises(ValueError):
        parse_think("extreme")
    assert format_parameters({"top_p": ["0.5"], "stop": ["a", "b"], "num_ctx": ["4096"], "use_mmap": ["true"]}) == \
        {"top_p": 0.5, "stop": ["a", "b"], "num_ctx": 4096, "use_mmap": True}
