"""The model / tool loop (agent/session.go:154-470), approvals (agent/approval.go), output budgets (session.go:879-1088) and
compaction (agent/compactor.go).

``Session.run`` sends the conversation with the tool schemas, executes the calls of the answer (asking first for the ones that
change things, unless their scope was allowed before), appends the results and repeats until an answer comes without calls,
the user refuses, or the round limit is reached.  Tool output is cut to a budget that follows the context window, keeping
head and tail around a marker that says how much is missing.  When the prompt has grown past three quarters of the window the
turns before the last user message are replaced by a summary the model writes itself.
"""
from __future__ import annotations

import json
import os
import threading
from dataclasses import dataclass, field
from typing import Any, Callable

from .tools import Registry, ToolError

DEFAULT_MAX_TOOL_ROUNDS = 100
MAX_TOOL_RESULT_CHARS = 60000
SMALL_CONTEXT = (8192, 6000)          # (context window up to, characters per tool result)
TINY_CONTEXT = (4096, 3200)
COMPACT_AT = 0.75                      # share of the context window at which older turns are summarised


def approximate_tokens(chars: int) -> int:
    """The usual four-characters-per-token estimate, for sizing decisions only."""
    return 0 if chars <= 0 else max(1, (chars + 3) // 4)


def truncate(content: str, max_chars: int, label: str = "tool output", head_pct: int = 75, hint: str = "") -> str:
    """At most ``max_chars`` characters of ``content``: the first ``head_pct`` percent of the budget and the rest from the end,
    with a marker in between that names what was dropped; ``max_chars`` <= 0 leaves only the marker."""
    hint = (" " + hint.strip().rstrip(".") + ".") if hint.strip() else ""
    total = len(content)
    if max_chars <= 0:
        return f"[{label} truncated: output omitted because the context is full; omitted ~{approximate_tokens(total)} tokens.{hint}]"
    if total <= max_chars:
        return content
    head = max_chars * head_pct // 100
    tail = max_chars - head
    marker = (f"\n\n[{label} truncated: showing first ~{approximate_tokens(head)} tokens and last ~{approximate_tokens(tail)} tokens; "
              f"omitted ~{approximate_tokens(total - head - tail)} tokens.{hint}]\n\n")
    return content[:head] + marker + (content[total - tail:] if tail else "")


def result_budget(context_window: int) -> int:
    if 0 < context_window <= TINY_CONTEXT[0]:
        return TINY_CONTEXT[1]
    if 0 < context_window <= SMALL_CONTEXT[0]:
        return SMALL_CONTEXT[1]
    return MAX_TOOL_RESULT_CHARS


@dataclass
class Approval:
    allow: bool
    allow_all: bool = False
    allow_scopes: list[str] = field(default_factory=list)
    reason: str = ""


class ApprovalState:
    """What the user has allowed for the rest of the session: everything, or single scopes (a tool, an exact shell command)."""

    def __init__(self):
        self._lock = threading.Lock()
        self.all = False
        self.scopes: set[str] = set()

    def allows(self, scope: str) -> bool:
        with self._lock:
            return self.all or scope in self.scopes

    def grant(self, approval: Approval) -> None:
        with self._lock:
            self.all = self.all or approval.allow_all
            self.scopes.update(approval.allow_scopes)


@dataclass
class RunResult:
    messages: list[dict[str, Any]]
    latest: dict[str, Any]
    working_dir: str
    stopped: str = "done"             # "done", "denied", "max_rounds"
    rounds: int = 0


class Session:
    def __init__(self, chat: Callable[..., dict[str, Any]], tools: Registry, *, approver: Callable[[list[dict[str, Any]], str], Approval] | None = None,
                 approvals: ApprovalState | None = None, working_dir: str | None = None, events: Callable[[str, dict[str, Any]], None] | None = None,
                 context_window: int = 0, skills=None):
        """``chat(**request)`` returns the body of a non-streaming ``/api/chat`` answer.  ``approver(calls, working_dir)`` decides about
        calls that need approval (None: they are refused).  ``events(kind, data)`` is told about every step."""
        self.chat, self.tools, self.approver = chat, tools, approver
        self.approvals = approvals or ApprovalState()
        self.working_dir = os.path.abspath(working_dir or os.getcwd())
        self.events = events or (lambda kind, data: None)
        self.context_window = context_window
        self.skills = skills

    # -- one run --------------------------------------------------------------------------------------
    def run(self, model: str, messages: list[dict[str, Any]], *, system: str = "", options: dict[str, Any] | None = None, think: Any = None,
            max_tool_rounds: int = 0, skill: str = "") -> RunResult:
        msgs = [dict(m) for m in messages]
        if system and not (msgs and msgs[0].get("role") == "system"):
            msgs.insert(0, {"role": "system", "content": system})
        if skill and self.skills is not None:          # a skill chosen by the caller enters as an already answered tool call
            call = {"id": "skill_0", "function": {"name": "skill", "arguments": {"name": skill}}}
            msgs += [{"role": "assistant", "content": "", "tool_calls": [call]}, {"role": "tool", "tool_name": "skill", "tool_call_id": "skill_0", "content": self.skills.load(skill)}]
        limit = DEFAULT_MAX_TOOL_ROUNDS if max_tool_rounds == 0 else max_tool_rounds
        latest: dict[str, Any] = {}
        rounds = 0
        while True:
            req: dict[str, Any] = {"model": model, "messages": list(msgs), "stream": False, "tools": self.tools.schemas()}
            if options:
                req["options"] = options
            if think is not None:
                req["think"] = think
            latest = self.chat(**req)
            answer = dict(latest.get("message") or {"role": "assistant", "content": ""})
            answer.setdefault("role", "assistant")
            msgs.append(answer)
            calls = answer.get("tool_calls") or []
            self.events("assistant", {"content": answer.get("content", ""), "thinking": answer.get("thinking", ""), "calls": len(calls)})
            if not calls:
                return RunResult(msgs, latest, self.working_dir, "done", rounds)
            rounds += 1
            if 0 < limit < rounds:
                msgs += [self._tool_message(c, "tool call skipped: the limit of consecutive tool rounds was reached") for c in calls]
                return RunResult(msgs, latest, self.working_dir, "max_rounds", rounds - 1)
            verdict = self._approve(calls)
            if not verdict.allow:
                why = "tool call denied by the user" + (f": {verdict.reason}" if verdict.reason else "")
                msgs += [self._tool_message(c, why) for c in calls]
                self.events("denied", {"reason": verdict.reason})
                return RunResult(msgs, latest, self.working_dir, "denied", rounds)
            budget = result_budget(self.context_window)
            for c in calls:
                msgs.append(self._tool_message(c, truncate(self._execute(c), budget, hint="Narrow the request (a file range, a filter) to see the rest")))
            msgs = self._maybe_compact(model, msgs, latest, options)

    # -- pieces ---------------------------------------------------------------------------------------
    @staticmethod
    def _args(call: dict[str, Any]) -> dict[str, Any]:
        a = (call.get("function") or {}).get("arguments")
        if isinstance(a, str):
            try:
                a = json.loads(a)
            except ValueError:
                a = {}
        return a if isinstance(a, dict) else {}

    @staticmethod
    def _tool_message(call: dict[str, Any], content: str) -> dict[str, Any]:
        return {"role": "tool", "tool_name": (call.get("function") or {}).get("name", ""), "tool_call_id": call.get("id", ""), "content": content}

    def _approve(self, calls: list[dict[str, Any]]) -> Approval:
        pending = []
        for c in calls:
            tool = self.tools.tools.get((c.get("function") or {}).get("name", ""))
            if tool is None or not tool.needs_approval:
                continue
            scope = tool.approval_scope(self._args(c))
            if not self.approvals.allows(scope) and not self.approvals.allows(tool.name):
                pending.append({"id": c.get("id", ""), "name": tool.name, "args": self._args(c), "scope": scope})
        if not pending:
            return Approval(True)
        if self.approver is None:
            return Approval(False, reason="no one is here to approve it")
        verdict = self.approver(pending, self.working_dir)
        if verdict.allow:
            self.approvals.grant(verdict)
        return verdict

    def _execute(self, call: dict[str, Any]) -> str:
        name = (call.get("function") or {}).get("name", "")
        self.events("tool_start", {"name": name, "args": self._args(call)})
        try:
            res = self.tools.execute(name, self._args(call), self.working_dir)
            if res.working_dir:
                self.working_dir = res.working_dir
            out = res.content
        except ToolError as e:
            out = f"error: {e}"
        except Exception as e:                      # a tool that blows up is the model's problem to read, not the session's
            out = f"error: {type(e).__name__}: {e}"
        self.events("tool_end", {"name": name, "chars": len(out)})
        return out

    def _maybe_compact(self, model: str, msgs: list[dict[str, Any]], latest: dict[str, Any], options: dict[str, Any] | None) -> list[dict[str, Any]]:
        """Past ``COMPACT_AT`` of the window: everything between the system message and the last user message becomes a summary."""
        if self.context_window <= 0:
            return msgs
        used = int(latest.get("prompt_eval_count") or 0) + int(latest.get("eval_count") or 0)
        used = max(used, approximate_tokens(sum(len(str(m.get("content") or "")) for m in msgs)))
        if used < COMPACT_AT * self.context_window:
            return msgs
        head = msgs[:1] if msgs and msgs[0].get("role") == "system" else []
        last_user = max((i for i, m in enumerate(msgs) if m.get("role") == "user"), default=-1)
        old = msgs[len(head):last_user] if last_user > len(head) else []
        if len(old) < 2:
            self.events("compaction_skipped", {"reason": "nothing old enough to summarise"})
            return msgs
        transcript = "\n".join(f"{m.get('role')}: {truncate(str(m.get('content') or ''), 2000, 'message')}" for m in old)
        ask = [{"role": "system", "content": "Summarise the conversation so far for your own later use: goals, decisions, facts learned from tools, "
                                              "open tasks. Be brief and concrete."}, {"role": "user", "content": transcript}]
        self.events("compaction_started", {"messages": len(old)})
        try:
            summary = (self.chat(model=model, messages=ask, stream=False, **({"options": options} if options else {})).get("message") or {}).get("content", "")
        except Exception as e:
            self.events("compaction_skipped", {"reason": str(e)})
            return msgs
        if not summary.strip():
            self.events("compaction_skipped", {"reason": "empty summary"})
            return msgs
        self.events("compacted", {"dropped": len(old), "summary_chars": len(summary)})
        return head + [{"role": "user", "content": "Summary of the conversation so far:\n" + summary.strip()}] + msgs[last_user:]
