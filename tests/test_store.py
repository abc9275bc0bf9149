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


def test_names_on_the_reference_table():
    """Validity, round trip, parts and shortest display of the reference's name tests (types/model/name_test.go:14-333)."""
    p80, p350 = "8" * 80, "3" * 350
    valid = {"": False, "_why/_the/_lucky:_stiff": True, "h/n/m:t": True, "host/namespace/model:tag": True, "host/namespace/model": False,
             "namespace/model": False, "model": False, f"{p80}/{p80}/{p80}:{p80}": True, f"{p350}/{p80}/{p80}:{p80}": True, "h/nn/mm:t": True,
             "m": False, "n/m:": False, "h/n/m": False, "@t": False, "m@d": False, "^": False, "mm:": False, "/nn/mm": False, "//": False,
             "//mm": False, "hh//": False, "//mm:@": False, "00@": False, "@": False, "-hh/nn/mm:tt": False, "hh/-nn/mm:tt": False,
             "hh/nn/-mm:tt": False, "hh/nn/mm:-tt": False, "host:https/namespace/model:tag": True, "host/name:space/model:tag": False,
             f"{p350}3/n/m:t": False, f"h/{p80}8/m:t": False, "h/n.s/m:t": False, "h./n/m:t": True}
    for s, want in valid.items():
        n = parse_name(s, fill_defaults=False)
        assert n.valid == want, s
        if want:
            assert str(n) == s
    parts = {"scheme://host:port/namespace/model:tag": ("host:port", "namespace", "model", "tag"),
             "host:port/namespace/model": ("host:port", "namespace", "model", ""), "namespace/model": ("", "namespace", "model", ""),
             "model": ("", "", "model", ""), "registry.ollama.ai/library/dolphin-mistral:7b-v2.6-dpo-laser-q6_K":
             ("registry.ollama.ai", "library", "dolphin-mistral", "7b-v2.6-dpo-laser-q6_K")}
    for s, want in parts.items():
        n = parse_name(s, fill_defaults=False)
        assert (n.host, n.namespace, n.model, n.tag) == want
    assert parse_name("namespace/model").filepath() == "registry.ollama.ai/namespace/model/latest"
    assert parse_name("model").filepath() == "registry.ollama.ai/library/model/latest"
    for s, want in {"registry.ollama.ai/library/model:latest": "model:latest", "registry.ollama.ai/namespace/model:tag": "namespace/model:tag",
                    "host/namespace/model:tag": "host/namespace/model:tag", "host/library/model:tag": "host/library/model:tag"}.items():
        assert parse_name(s).display() == want


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


def _cmds(text):
    return [("model" if c.name == "from" and not c.is_parameter else c.name, c.args) for c in parse_modelfile(text).commands]


def test_modelfile_on_the_reference_tables():
    """Commands and values of the reference's parser tests (parser/parser_test.go:123-766): trimming, quoting over several lines,
    quotes inside a value, parameters, messages, comments, UTF-16 input and the inputs that must be refused."""
    ok = [
        ('FROM "FOO  BAR  "', [("model", "FOO  BAR  ")]),
        ('FROM "FOO BAR"\nPARAMETER param1 value1', [("model", "FOO BAR"), ("param1", "value1")]),
        ("FROM     FOOO BAR    ", [("model", "FOOO BAR")]),
        ("FROM /what/is/the path ", [("model", "/what/is/the path")]),
        ("FROM llama3:7b-instruct-q4_K_M", [("model", "llama3:7b-instruct-q4_K_M")]),
        ("PARAMETER param1 value1\nFROM foo", [("param1", "value1"), ("model", "foo")]),
        ("PARAMETER what the \nFROM lemons make lemonade ", [("what", "the"), ("model", "lemons make lemonade")]),
        ('\nFROM "     model 1"\nADAPTER      adapter3\nLICENSE "MIT       "\nPARAMETER param1        value1\nTEMPLATE """   {{ a }}\n\n{{ b }}   """    \n',
         [("model", "     model 1"), ("adapter", "adapter3"), ("license", "MIT       "), ("param1", "value1"), ("template", "   {{ a }}\n\n{{ b }}   ")]),
        ("\nFROM foo\nMESSAGE system You are a file parser. Always parse things.", [("model", "foo"), ("message", "system: You are a file parser. Always parse things.")]),
        ('\nFROM foo\nMESSAGE system """\nYou are a multiline file parser.\n"""\n\t\t\t', [("model", "foo"), ("message", "system: \nYou are a multiline file parser.\n")]),
        ('\nFROM foo\nSYSTEM """\nThis is a\nmultiline system.\n"""\n\t\t\t', [("model", "foo"), ("system", "\nThis is a\nmultiline system.\n")]),
        ('\nFROM foo\nSYSTEM """This is a\nmultiline system."""\n\t\t\t', [("model", "foo"), ("system", "This is a\nmultiline system.")]),
        ('\nFROM foo\nSYSTEM """\nThis is a multiline system with "quotes".\n"""\n', [("model", "foo"), ("system", '\nThis is a multiline system with "quotes".\n')]),
        ('\nFROM foo\nSYSTEM """\nUse """three quotes""" inside a line\n"""\n', [("model", "foo"), ("system", '\nUse """three quotes""" inside a line\n')]),
        ('\nFROM foo\nSYSTEM """"""\n', [("model", "foo"), ("system", "")]),
        ('\nFROM foo\nSYSTEM ""\n', [("model", "foo"), ("system", "")]),
        ('\nFROM foo\nSYSTEM "\'"\n', [("model", "foo"), ("system", "'")]),
        ('\nFROM foo\nSYSTEM """\'\'"\'""\'""\'"\'\'\'\'\'""\'""\'"""\n', [("model", "foo"), ("system", '\'\'"\'""\'""\'"\'\'\'\'\'""\'""\'')]),
        ('\nFROM foo\nTEMPLATE """\n{{ .Prompt }}\n"""', [("model", "foo"), ("template", "\n{{ .Prompt }}\n")]),
        ("\n# comment\nFROM foo\n\t", [("model", "foo")]),
        ("\nFROM base\nDRAFT ./assistant\n", [("model", "base"), ("draft", "./assistant")]),
        ("FROM test\n\tSYSTEM 你好👋", [("model", "test"), ("system", "你好👋")]),
    ]
    for text, want in ok:
        assert _cmds(text) == want, text
    params = {"numa true": ("numa", "true"), "top_p 1.0": ("top_p", "1.0"), "stop ### User:": ("stop", "### User:"), "stop ### User: ": ("stop", "### User:"),
              'stop "### User:"': ("stop", "### User:"), 'stop "### User: "': ("stop", "### User: "), 'stop """### User:"""': ("stop", "### User:"),
              'stop """### User:\n"""': ("stop", "### User:\n"), "stop <|endoftext|>": ("stop", "<|endoftext|>"), "stop </s>": ("stop", "</s>")}
    for line, want in params.items():
        assert _cmds(f"FROM foo\nPARAMETER {line}\n") == [("model", "foo"), want], line
    for bad in ("", "PARAMETER param1 value1", "\nFROM foo\nPARAMETER param1\n", "\nFROM foo\nBADCOMMAND param1 value1\n", "\nFROM foo\nMESSAGE badguy I'm a bad guy!\n",
                "\nFROM foo\nMESSAGE system\n", "\nFROM foo\nMESSAGE system", '\nFROM foo\nSYSTEM """This is a multiline system.""\n\t\t\t', '\nFROM foo\nSYSTEM "\n\t\t\t'):
        with pytest.raises(ModelfileError):
            parse_modelfile(bad)
    text = "FROM bob\nPARAMETER param1 1\nPARAMETER param2 4096\nSYSTEM You are a utf16 file. 你好👋\n"
    want = [("model", "bob"), ("param1", "1"), ("param2", "4096"), ("system", "You are a utf16 file. 你好👋")]
    for data in (b"\xff\xfe" + text.encode("utf-16-le"), b"\xfe\xff" + text.encode("utf-16-be"), b"\xef\xbb\xbf" + text.encode(), text.encode()):
        assert _cmds(data) == want
    # serialise -> parse gives the same commands (TestParseFileFormatParseFile)
    for text in ('\nFROM foo\nADAPTER adapter1\nLICENSE """\nVery long and boring legal text.\nBlah blah blah.\n"Oh look, a quote!"\n"""\n\nPARAMETER param1 value1\nTEMPLATE template1\n'
                 'MESSAGE system """\nYou are a store greeter. Always respond with "Hello!".\n"""\nMESSAGE user Hey there!\n', '\nFROM foo\nSYSTEM ""\n'):
        assert _cmds(str(parse_modelfile(text))) == _cmds(text)
    req = parse_modelfile("FROM test\nPARAMETER temperature 0.5\nPARAMETER top_k 1\nSYSTEM You are a bot.\nLICENSE license1\nLICENSE license2\n"
                          "MESSAGE user Hello there!\nMESSAGE assistant Hi! How are you?\n").create_request()
    assert req == {"from": "test", "license": ["license1", "license2"], "system": "You are a bot.", "parameters": {"temperature": 0.5, "top_k": 1},
                   "messages": [{"role": "user", "content": "Hello there!"}, {"role": "assistant", "content": "Hi! How are you?"}]}


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
    # a delete removes only the deleted manifest's own unused layers: a blob no manifest names (an upload waiting for
    # its create, a layer of a pull in progress) stays, and so does one that another manifest still uses
    assert os.path.exists(orphan.path()) and os.path.exists(a.path())
    M.delete_model(parse_name("me/other"))
    assert not os.path.exists(a.path()) and not os.path.exists(cfg.path()) and os.path.exists(orphan.path())
    assert M.prune_layers() == 1 and not os.path.exists(orphan.path())             # the start-up sweep takes the orphan
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
    cases = {"1.2.3.4": "http://1.2.3.4:11434", ":1234": "http://:1234", "example.com:99": "http://example.com:99",
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


def test_envconfig_on_the_reference_tables(monkeypatch):
    """Hosts, booleans, unsigned values, durations, quoting and log levels of envconfig/config_test.go:13-330 of the reference."""
    hosts = {"": "http://127.0.0.1:11434", "1.2.3.4": "http://1.2.3.4:11434", ":1234": "http://:1234", "1.2.3.4:1234": "http://1.2.3.4:1234",
             "example.com": "http://example.com:11434", ":0": "http://:0", ":66000": "http://:11434", ":-1": "http://:11434",
             "[::1]": "http://[::1]:11434", "[::]": "http://[::]:11434", "::1": "http://[::1]:11434", "[::1]:1337": "http://[::1]:1337",
             " 1.2.3.4 ": "http://1.2.3.4:11434", '"1.2.3.4"': "http://1.2.3.4:11434", ' " 1.2.3.4 " ': "http://1.2.3.4:11434",
             "'1.2.3.4'": "http://1.2.3.4:11434", "http://1.2.3.4": "http://1.2.3.4:80", "http://1.2.3.4:4321": "http://1.2.3.4:4321",
             "https://1.2.3.4": "https://1.2.3.4:443", "https://example.com/ollama": "https://example.com:443/ollama",
             "ollama.com": "https://ollama.com:443"}
    for v, want in hosts.items():
        monkeypatch.setenv("OLLAMA_HOST", v)
        assert str(envconfig.host()) == want, v
    connectable = {"": "http://127.0.0.1:11434", "127.0.0.1:1234": "http://127.0.0.1:1234", "0.0.0.0": "http://127.0.0.1:11434",
                   "0.0.0.0:1234": "http://127.0.0.1:1234", "[::]": "http://[::1]:11434", "[::]:1234": "http://[::1]:1234",
                   "[::1]:1234": "http://[::1]:1234", "192.168.1.5:8080": "http://192.168.1.5:8080", "example.com": "http://example.com:11434",
                   "https://0.0.0.0:4321": "https://127.0.0.1:4321", ":1234": "http://127.0.0.1:1234"}
    for v, want in connectable.items():
        monkeypatch.setenv("OLLAMA_HOST", v)
        assert str(envconfig.connectable_host()) == want, v
    for v, want in {"": False, "true": True, "false": False, "1": True, "0": False, "random": True, "something": True}.items():
        monkeypatch.setenv("OLLAMA_NOPRUNE", v)
        assert envconfig.no_prune() is want, v
    for v, want in {"0": 0, "1": 1, "1337": 1337, "": 512, "-1": 512, "0o10": 512, "0x10": 512, "string": 512}.items():
        monkeypatch.setenv("OLLAMA_MAX_QUEUE", v)
        assert envconfig.max_queue() == want, v
    inf = math.inf
    for v, want in {"": 300, "1s": 1, "1m": 60, "1h": 3600, "5m0s": 300, "1h2m3s": 3723, "0": 0, "60": 60, "3600": 3600, "-0": 0, "-1": inf,
                    "-1m": inf, " ": 300, "???": 300, "1d": 300, "1y": 300, "1w": 300}.items():
        monkeypatch.setenv("OLLAMA_KEEP_ALIVE", v)
        assert envconfig.keep_alive() == want, v
    for v, want in {"": 300, "1s": 1, "5m0s": 300, "1h2m3s": 3723, "0": inf, "60": 60, "-0": inf, "-1": inf, "-1m": inf, "???": 300, "1d": 300}.items():
        monkeypatch.setenv("OLLAMA_LOAD_TIMEOUT", v)
        assert envconfig.load_timeout() == want, v
    for v, want in {"value": "value", " value ": "value", " 'value' ": "value", ' "value" ': "value", " ' value ' ": " value ", ' " value " ': " value "}.items():
        monkeypatch.setenv("OLLAMA_LLM_LIBRARY", v)
        assert envconfig.llm_library() == want, v
    for v, want in {"": 20, "false": 20, "f": 20, "0": 20, "true": 10, "t": 10, "1": 10, "2": 5, "-1": 30, "-2": 40}.items():
        monkeypatch.setenv("OLLAMA_DEBUG", v)
        assert envconfig.log_level() == want, v


def test_no_cloud_from_environment_or_config_file(monkeypatch, tmp_path):
    """envconfig/config_test.go:332-420 of the reference."""
    for env, content, disabled, source in (("", None, False, "none"), ("1", None, True, "env"), ("", '{"disable_ollama_cloud": true}', True, "config"),
                                           ("1", '{"disable_ollama_cloud": true}', True, "both"), ("", '{"disable_ollama_cloud": false}', False, "none"),
                                           ("", "{invalid json", False, "none")):
        home = tmp_path / f"h{abs(hash((env, content)))}"
        (home / ".ollama").mkdir(parents=True)
        if content is not None:
            (home / ".ollama" / "server.json").write_text(content)
        monkeypatch.setenv("HOME", str(home))
        monkeypatch.setenv("OLLAMA_NO_CLOUD", env)
        assert envconfig.no_cloud() is disabled and envconfig.no_cloud_source() == source


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
