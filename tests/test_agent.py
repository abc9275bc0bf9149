"""Agent runtime with a scripted model (the reference tests its session the same way, agent/session_test.go: a fake chat client
that answers from a list, real tools in a temporary directory)."""
import os

import pytest

from ollama_b200.agent import Approval, Session, default_registry, truncate
from ollama_b200.agent.session import approximate_tokens, result_budget
from ollama_b200.agent.skills import SkillCatalog


def call(name, cid="c1", **args):
    return {"id": cid, "function": {"name": name, "arguments": args}}


class Script:
    def __init__(self, answers):
        self.answers, self.requests = list(answers), []

    def __call__(self, **req):
        self.requests.append(req)
        a = self.answers.pop(0)
        msg = a if "role" in a else {"role": "assistant", **a}
        return {"message": msg, "prompt_eval_count": a.get("_used", 10), "eval_count": 5, "done": True}


def test_loop_runs_tools_until_the_model_answers(tmp_path):
    (tmp_path / "notes.txt").write_text("alpha\nbeta\ngamma\n")
    script = Script([{"content": "", "tool_calls": [call("read_file", path="notes.txt", offset=2, limit=1), call("list_dir", "c2")]},
                     {"content": "", "tool_calls": [call("edit_file", path="notes.txt", old_string="beta", new_string="BETA")]},
                     {"content": "done"}])
    asked = []
    s = Session(script, default_registry(), working_dir=str(tmp_path), approver=lambda calls, cwd: asked.append(calls) or Approval(True, allow_scopes=["edit_file"]))
    r = s.run("m", [{"role": "user", "content": "fix the notes"}], system="be careful")
    assert r.stopped == "done" and r.rounds == 2 and (tmp_path / "notes.txt").read_text() == "alpha\nBETA\ngamma\n"
    roles = [m["role"] for m in r.messages]
    assert roles == ["system", "user", "assistant", "tool", "tool", "assistant", "tool", "assistant"]
    assert r.messages[3]["content"].strip() == "2\tbeta\n[1 more lines; continue with offset=3]".strip() and r.messages[4]["content"] == "notes.txt"
    assert r.messages[6]["tool_call_id"] == "c1" and "replaced 1 occurrence" in r.messages[6]["content"]
    assert len(asked) == 1 and asked[0][0]["name"] == "edit_file"            # reading needs no approval, the edit does
    assert [t["function"]["name"] for t in script.requests[0]["tools"]] == ["bash", "edit_file", "list_dir", "read_file", "write_file"]
    # "always allow" for the tool: the next edit goes through unasked
    script.answers = [{"content": "", "tool_calls": [call("edit_file", path="notes.txt", old_string="alpha", new_string="A")]}, {"content": "ok"}]
    s.run("m", r.messages + [{"role": "user", "content": "again"}])
    assert len(asked) == 1 and (tmp_path / "notes.txt").read_text().startswith("A\n")


def test_denial_round_limit_unknown_tool_and_failing_tool(tmp_path):
    s = Session(Script([{"content": "", "tool_calls": [call("bash", command="rm -rf /")]}]), default_registry(), working_dir=str(tmp_path),
                approver=lambda calls, cwd: Approval(False, reason="too dangerous"))
    r = s.run("m", [{"role": "user", "content": "clean up"}])
    assert r.stopped == "denied" and "denied by the user: too dangerous" in r.messages[-1]["content"]
    r = Session(Script([{"content": "", "tool_calls": [call("bash", command="ls")]}]), default_registry(), working_dir=str(tmp_path)).run("m", [{"role": "user", "content": "x"}])
    assert r.stopped == "denied" and "no one is here" in r.messages[-1]["content"]
    loop = Script([{"content": "", "tool_calls": [call("list_dir")]}] * 5)
    r = Session(loop, default_registry(), working_dir=str(tmp_path)).run("m", [{"role": "user", "content": "x"}], max_tool_rounds=3)
    assert r.stopped == "max_rounds" and r.rounds == 3 and "limit of consecutive tool rounds" in r.messages[-1]["content"] and len(loop.requests) == 4
    script = Script([{"content": "", "tool_calls": [call("nope"), call("read_file", "c2", path="missing.txt"), call("edit_file", "c3", path="missing.txt")]}, {"content": "hm"}])
    r = Session(script, default_registry(), working_dir=str(tmp_path), approver=lambda c, d: Approval(True)).run("m", [{"role": "user", "content": "x"}])
    assert [m["content"][:22] for m in r.messages if m["role"] == "tool"] == ["error: unknown tool: n", "error: cannot read " + str(tmp_path)[:3], "error: old_string and "]


def test_shell_tool_moves_the_working_directory_and_scopes_approval_to_the_command(tmp_path):
    (tmp_path / "sub").mkdir()
    asked = []

    def approver(calls, cwd):
        asked.append([c["scope"] for c in calls])
        return Approval(True, allow_scopes=[c["scope"] for c in calls])

    script = Script([{"content": "", "tool_calls": [call("bash", command="cd sub && echo hi && false")]}, {"content": "", "tool_calls": [call("bash", command="pwd")]},
                     {"content": "", "tool_calls": [call("bash", command="cd sub && echo hi && false")]}, {"content": "fin"}])
    s = Session(script, default_registry(), working_dir=str(tmp_path), approver=approver)
    (tmp_path / "sub" / "sub").mkdir()
    r = s.run("m", [{"role": "user", "content": "go"}])
    outs = [m["content"] for m in r.messages if m["role"] == "tool"]
    assert outs[0] == "hi\n[exit code 1]" and outs[1].strip() == str(tmp_path / "sub") and r.working_dir == str(tmp_path / "sub" / "sub")
    assert asked == [["bash\x00cd sub && echo hi && false"], ["bash\x00pwd"]]          # the repeated command was not asked about again


def test_output_budget_and_markers():
    assert approximate_tokens(0) == 0 and approximate_tokens(1) == 1 and approximate_tokens(9) == 3
    assert result_budget(0) == 60000 and result_budget(8192) == 6000 and result_budget(4096) == 3200 and result_budget(32768) == 60000
    text = "a" * 100 + "b" * 100
    out = truncate(text, 40, hint="ask for less")
    assert out.startswith("a" * 30 + "\n\n[tool output truncated: showing first ~8 tokens and last ~3 tokens; omitted ~40 tokens. ask for less.]\n\n") and out.endswith("b" * 10)
    assert truncate(text, 500) == text and truncate(text, 0).startswith("[tool output truncated: output omitted because the context is full; omitted ~50 tokens.")


def test_compaction_replaces_old_turns_with_a_summary(tmp_path):
    events = []
    script = Script([{"content": "", "tool_calls": [call("list_dir")], "_used": 900}, {"content": "SUMMARY: the user wants a listing"}, {"content": "all done"}])
    s = Session(script, default_registry(), working_dir=str(tmp_path), context_window=1000, events=lambda k, d: events.append(k))
    history = [{"role": "system", "content": "sys"}, {"role": "user", "content": "first"}, {"role": "assistant", "content": "answer one"},
               {"role": "user", "content": "second"}, {"role": "assistant", "content": "answer two"}, {"role": "user", "content": "list it"}]
    r = s.run("m", history)
    assert r.stopped == "done" and "compacted" in events
    assert [m["role"] for m in r.messages] == ["system", "user", "user", "assistant", "tool", "assistant"]
    assert r.messages[1]["content"].startswith("Summary of the conversation so far:\nSUMMARY") and r.messages[2]["content"] == "list it"
    assert "first" in script.requests[1]["messages"][1]["content"] and "tools" not in script.requests[1]


def test_skills_catalog_and_synthetic_call(tmp_path):
    d = tmp_path / "skills" / "release"
    d.mkdir(parents=True)
    (d / "SKILL.md").write_text("---\nname: release-notes\ndescription: Write release notes\n---\nCollect the merged changes, then group them.\n")
    (tmp_path / "skills" / "broken").mkdir()
    cat = SkillCatalog([str(tmp_path / "skills"), str(tmp_path / "absent")])
    assert cat.names() == ["release-notes"] and "Write release notes" in cat.describe() and "Collect the merged changes" in cat.load("release-notes")
    with pytest.raises(KeyError):
        cat.load("nope")
    reg = default_registry(cat)
    assert "skill" in reg.names() and "release-notes" in reg.tools["skill"].description
    script = Script([{"content": "ok"}])
    r = Session(script, reg, working_dir=str(tmp_path), skills=cat).run("m", [{"role": "user", "content": "notes please"}], skill="release-notes")
    sent = script.requests[0]["messages"]
    assert [m["role"] for m in sent] == ["user", "assistant", "tool"] and sent[1]["tool_calls"][0]["function"]["name"] == "skill" and "group them" in sent[2]["content"]
    assert r.stopped == "done" and os.path.isdir(r.working_dir)
