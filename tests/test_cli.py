"""Command line against a live server (uvicorn in a thread, CPU backend, temp model store)."""
import io
import json
import os
import socket
import threading
import time
from contextlib import redirect_stderr, redirect_stdout

import pytest


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    root = tmp_path_factory.mktemp("cli_store")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    keys = ("OLLAMA_MODELS", "B200_DEVICE", "OLLAMA_CONTEXT_LENGTH", "OLLAMA_HOST")
    old = {k: os.environ.get(k) for k in keys}
    os.environ.update(OLLAMA_MODELS=str(root), B200_DEVICE="cpu", OLLAMA_CONTEXT_LENGTH="256", OLLAMA_HOST=f"127.0.0.1:{port}")
    import uvicorn

    from ollama_b200.models.synth import write_synthetic_gguf
    from ollama_b200.server.routes import create_app
    write_synthetic_gguf(str(root / "m.gguf"), "tiny-llama", "F32")
    (root / "Modelfile").write_text('FROM ./m.gguf\nTEMPLATE "{{ .Prompt }}"\nPARAMETER temperature 0\nPARAMETER num_predict 5\nSYSTEM be brief\n')
    srv = uvicorn.Server(uvicorn.Config(create_app(), host="127.0.0.1", port=port, log_level="warning"))
    t = threading.Thread(target=srv.run, daemon=True)
    t.start()
    for _ in range(200):
        if srv.started:
            break
        time.sleep(0.05)
    yield root
    srv.should_exit = True
    t.join(timeout=10)
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def run_cli(*argv):
    from ollama_b200.cli.main import main
    out, err = io.StringIO(), io.StringIO()
    with redirect_stdout(out), redirect_stderr(err):
        rc = main(list(argv))
    return rc, out.getvalue(), err.getvalue()


def test_create_list_show_run_cp_rm(server, monkeypatch):
    monkeypatch.setattr("sys.stdin", io.StringIO(""))          # not a tty: `run` takes the prompt from argv only
    rc, out, err = run_cli("create", "tiny", "-f", str(server / "Modelfile"))
    assert rc == 0 and "success" in err
    rc, out, _ = run_cli("list")
    assert rc == 0 and out.splitlines()[0].split() == ["NAME", "ID", "SIZE", "MODIFIED"] and "tiny:latest" in out
    rc, out, _ = run_cli("show", "tiny")
    assert rc == 0 and "architecture" in out and "llama" in out
    rc, out, _ = run_cli("show", "tiny", "--system")
    assert out.strip() == "be brief"
    rc, out, err = run_cli("run", "tiny", "<t300><t301>", "--verbose")
    assert rc == 0 and out.count("<t") == 5 and "eval rate" in err
    rc, out, _ = run_cli("ps")
    assert rc == 0 and "tiny:latest" in out and "CPU" in out
    rc, out, _ = run_cli("cp", "tiny", "tiny2")
    assert rc == 0
    rc, out, _ = run_cli("rm", "tiny2")
    assert rc == 0 and "deleted" in out
    rc, out, err = run_cli("rm", "tiny2")
    assert rc == 1 and "not found" in err
    rc, _, _ = run_cli("stop", "tiny")
    assert rc == 0


def test_create_refuses_a_draft_that_is_the_model_itself(server):
    """parser/parser_test.go:93-121 of the reference: DRAFT and FROM must not be the same local path."""
    (server / "SameDraft").write_text("FROM ./m.gguf\nDRAFT ./m.gguf\n")
    with pytest.raises(SystemExit, match="DRAFT must not reference the same local path as FROM"):
        run_cli("create", "same", "-f", str(server / "SameDraft"))


def test_bench_formats(server):
    run_cli("create", "tiny", "-f", str(server / "Modelfile"))
    rc, out, _ = run_cli("bench", "--model", "tiny", "--epochs", "2", "--max-tokens", "4", "--prompt-tokens", "8", "--format", "json")
    res = json.loads(out)
    assert rc == 0 and res[0]["model"] == "tiny" and res[0]["generate_tok_s"] > 0 and res[0]["ttft_ms"] > 0
    rc, out, _ = run_cli("bench", "--model", "tiny", "--epochs", "1", "--max-tokens", "3")
    assert "BenchmarkModel/name=tiny/step=generate" in out and "token/sec" in out


def test_repl_commands(server, monkeypatch):
    from ollama_b200.api.client import Client
    from ollama_b200.cli.main import Repl
    run_cli("create", "tiny", "-f", str(server / "Modelfile"))
    lines = iter(["/set parameter num_predict 3", "/set system terse", '"""<t300>', '<t301>"""', "/clear", "/bogus", "/bye"])
    monkeypatch.setattr("builtins.input", lambda prompt="": next(lines))
    out = io.StringIO()
    r = Repl(Client(), "tiny", {}, "", None, None, False)
    with redirect_stdout(out):
        r.loop()
    text = out.getvalue()
    assert r.opts == {"num_predict": 3} and r.system == "terse" and r.messages == []
    assert text.count("<t") == 3 and "Unknown command '/bogus'" in text and "Cleared session context" in text


def test_repl_load_save_and_history(server, monkeypatch, tmp_path):
    """cmd/interactive.go:209-278 (/load, /save) and readline/history.go:24-103 (100 entries, rewritten after every line,
    OLLAMA_NOHISTORY)."""
    from ollama_b200.api.client import Client
    from ollama_b200.cli import lineedit
    from ollama_b200.cli.main import Repl
    run_cli("create", "tiny", "-f", str(server / "Modelfile"))
    monkeypatch.setattr(lineedit, "history_path", lambda: str(tmp_path / "hist" / "history"))
    lines = iter(["/set parameter num_predict 2", "/set system brief", "<t300>", "/save tiny-session", "/load nope", "/load tiny-session", "/save", "/set nohistory",
                  "secret", "/bye"])
    monkeypatch.setattr("builtins.input", lambda prompt="": next(lines))
    out = io.StringIO()
    r = Repl(Client(), "tiny", {}, "", None, None, False)
    with redirect_stdout(out):
        r.loop()
    text = out.getvalue()
    assert "Created new model 'tiny-session'" in text and "Couldn't find model 'nope'" in text and "Loading model 'tiny-session'" in text
    assert "Usage:\n  /save <modelname>" in text and r.model == "tiny-session"
    info = Client().show("tiny-session")
    assert info["system"] == "brief" and "num_predict" in info["parameters"] and [m["role"] for m in info["messages"]] == ["user", "assistant"]
    saved = open(tmp_path / "hist" / "history", encoding="utf-8").read().splitlines()
    assert saved[:3] == ["/set parameter num_predict 2", "/set system brief", "<t300>"] and "secret" not in saved and "/bye" not in saved
    # the file keeps the newest entries up to the limit, skips repeats, and is not touched when history is off
    h = lineedit.History(str(tmp_path / "h2"), limit=3)
    for x in ("a", "b", "b", "c", "d"):
        h.add(x)
    assert h.entries == ["b", "c", "d"] and lineedit.History(str(tmp_path / "h2"), limit=3).entries == ["b", "c", "d"]
    monkeypatch.setenv("OLLAMA_NOHISTORY", "1")
    off = lineedit.History(str(tmp_path / "h3"))
    off.add("x")
    assert off.entries == [] and not (tmp_path / "h3").exists()
    assert lineedit.complete("/s", "/s") == ["/set ", "/show ", "/save "] and lineedit.complete("no", "/set no") == ["nohistory ", "nowordwrap ", "noformat ", "nothink "]
    assert lineedit.complete("te", "/show te") == ["template"] and lineedit.complete("x", "hello x") == []


def test_launch_wires_tools_to_the_server(server, monkeypatch, tmp_path):
    """cmd/launch: environment of Claude Code (claude.go:63-83), overrides of Codex (codex.go:35-49, 174-204), inline configuration of
    OpenCode (opencode.go:289-386), settings edit of Droid (droid.go:67-150), the saved choice (cmd/config/config.go) and the pickers."""
    from ollama_b200.api.client import Client
    from ollama_b200.cli import launch as L
    from ollama_b200.cli import tui
    run_cli("create", "tiny", "-f", str(server / "Modelfile"))
    monkeypatch.setenv("HOME", str(tmp_path))
    monkeypatch.setenv("OLLAMA_HOST", os.environ.get("OLLAMA_HOST", "127.0.0.1:11434"))
    host = L.host_url()
    assert host.startswith("http://127.0.0.1:")
    env = L.claude_env("m1", [])
    assert env["ANTHROPIC_BASE_URL"] == host and env["ANTHROPIC_AUTH_TOKEN"] == "ollama" and env["ANTHROPIC_DEFAULT_SONNET_MODEL"] == "m1" and env["ANTHROPIC_API_KEY"] == ""
    args = L.codex_args("m1", ["exec", "hi"])
    assert args[:2] == ["-c", 'model_provider="ollama-launch"'] and f'model_providers.ollama-launch.base_url="{host}/v1/"' in args and args[-4:] == ["-m", "m1", "exec", "hi"]
    with pytest.raises(L.LaunchError):
        L.codex_args("m1", ["-c", "model_providers.x.base_url=evil"])
    cfg = json.loads(L.opencode_env("m1", [L.LaunchModel("m1", ["thinking", "vision"], 8192, 4096), L.LaunchModel("m2")])["OPENCODE_CONFIG_CONTENT"])
    prov = cfg["provider"]["ollama"]
    assert cfg["model"] == "ollama/m1" and prov["options"]["baseURL"] == host + "/v1" and prov["models"]["m1"]["limit"] == {"context": 8192, "output": 4096}
    assert prov["models"]["m1"]["reasoning"] is True and prov["models"]["m1"]["modalities"]["input"] == ["text", "image"] and prov["models"]["m2"] == {"name": "m2"}
    # droid: our entries replace those of an earlier launch and go in front of the user's own
    sp = tmp_path / ".factory" / "settings.json"
    sp.parent.mkdir()
    sp.write_text(json.dumps({"theme": "dark", "customModels": [{"model": "old", "apiKey": "ollama"}, {"model": "mine", "apiKey": "sk-1"}],
                              "sessionDefaultSettings": {"reasoningEffort": "turbo"}}))
    L.droid_configure("m1", [L.LaunchModel("m1", ["vision"]), L.LaunchModel("m2", max_output_tokens=100)])
    st = json.loads(sp.read_text())
    assert [m["model"] for m in st["customModels"]] == ["m1", "m2", "mine"] and st["theme"] == "dark" and (tmp_path / ".factory" / "settings.json.bak").exists()
    assert st["customModels"][0] == {"model": "m1", "displayName": "m1", "baseUrl": host + "/v1", "apiKey": "ollama", "provider": "generic-chat-completion-api",
                                     "maxOutputTokens": 64000, "supportsImages": True, "id": "custom:m1-0", "index": 0}
    assert st["customModels"][1]["maxOutputTokens"] == 100 and st["sessionDefaultSettings"] == {"reasoningEffort": "none", "model": "custom:m1-0"}
    # the command: pick from the list (piped input), remember the choice, dry run, missing tool, unknown names
    out = io.StringIO()
    assert L.launch(Client(), None, None, [], choose_only=True, inp=io.StringIO("claude\ntiny\n"), out=out) == 0
    assert L.saved_models("claude") == ["tiny:latest"] and "will use tiny:latest" in out.getvalue()
    out = io.StringIO()
    assert L.launch(Client(), "claude", None, ["-p", "hi"], dry_run=True, out=out) == 0
    line = out.getvalue().strip().splitlines()[-1]
    assert "ANTHROPIC_BASE_URL=" + host in line and line.endswith("claude --model tiny:latest -p hi")
    ran = []
    monkeypatch.setattr(L.Integration, "find", lambda self: "/usr/bin/" + self.binary)
    assert L.launch(Client(), "codex", "tiny", [], run=lambda cmd, env: ran.append((cmd, env.get("OPENAI_API_KEY"))) or 0, out=io.StringIO()) == 0
    assert ran[0][0][0] == "/usr/bin/codex" and ran[0][0][-2:] == ["-m", "tiny"] and ran[0][1] == "ollama"
    monkeypatch.setattr(L.Integration, "find", lambda self: None)
    out = io.StringIO()
    assert L.launch(Client(), "droid", "tiny", [], out=out) == 1 and "Droid is not installed" in out.getvalue() and "ollama launch droid" in out.getvalue()
    assert L.launch(Client(), "nope", "tiny", [], out=io.StringIO()) == 1 and L.launch(Client(), "claude", "absent", [], out=io.StringIO()) == 1
    # selector keys
    st = tui.SelectorState([tui.Item("alpha", "first"), tui.Item("beta"), tui.Item("gamma", "has alpha in its text")], height=2)
    assert st.key("down") is None and st.current.name == "beta" and st.key("down") is None and st.current.name == "gamma" and st.offset == 1
    for ch in "alp":
        st.key(ch)
    assert [i.name for i in st.visible] == ["alpha", "gamma"] and st.current.name == "alpha" and st.key("\r") == "pick"
    st.key("x")
    assert st.visible == [] and st.key("\r") is None and st.key("\x7f") is None and len(st.visible) == 2 and st.key("\x1b") == "cancel"
    assert tui.confirm("ok?", inp=io.StringIO("y\n"), out=io.StringIO()) and not tui.confirm("ok?", inp=io.StringIO("\n"), out=io.StringIO())
    with pytest.raises(tui.Cancelled):
        tui.select("pick", [tui.Item("a")], inp=io.StringIO("zzz\n"), out=io.StringIO())
    rc, _, err_text = run_cli("launch", "claude", "--model", "tiny", "--dry-run", "--", "--print", "hello")
    assert rc == 0 and err_text.strip().endswith("claude --model tiny --print hello")


def test_prompt_lines_carry_image_files(tmp_path, capsys):
    """cmd/interactive.go:605-644: paths of image files inside a prompt leave the text and travel as images; names of files that do
    not exist stay; a file of another kind behind an image extension is refused."""
    import base64

    from ollama_b200.cli.main import extract_media
    png = tmp_path / "a pic.png"
    png.write_bytes(b"\x89PNG\r\n\x1a\n" + b"\0" * 32)
    jpg = tmp_path / "b.JPG"
    jpg.write_bytes(b"\xff\xd8\xff\xe0" + b"\0" * 32)
    esc = str(png).replace(" ", "\\ ")
    text, images = extract_media(f"compare {esc} with '{jpg}' and /no/such/file.png please")
    assert text == "compare  with  and /no/such/file.png please"
    assert [base64.b64decode(i)[:4] for i in images] == [b"\x89PNG", b"\xff\xd8\xff\xe0"]
    assert "Added image" in capsys.readouterr().err
    assert extract_media("no files here") == ("no files here", [])
    fake = tmp_path / "notes.png"
    fake.write_text("just text")
    with pytest.raises(ValueError, match="invalid file type"):
        extract_media(f"look at {fake}")
    wav = tmp_path / "s.wav"
    wav.write_bytes(b"RIFF\0\0\0\0WAVEfmt " + b"\0" * 16)
    assert len(extract_media(f"{wav} transcribe")[1]) == 1
