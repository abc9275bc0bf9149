"""Agent runtime: a model that works through tools (shell, files, skills) until it has an answer.

Counterpart of the reference's ``agent`` package (agent/session.go, registry.go, approval.go, compactor.go, skills.go,
agent/tools/*.go) on top of this repository's API client: :class:`Session` runs the model / tool loop, :class:`Registry`
holds the tools, :class:`ApprovalState` remembers what the user allowed, :func:`truncate` keeps tool output inside the
context budget, and the compactor replaces old turns by a summary when the context fills up.
"""
from .session import Approval, ApprovalState, RunResult, Session, approximate_tokens, truncate  # noqa: F401
from .tools import Registry, Tool, ToolResult, default_registry  # noqa: F401
