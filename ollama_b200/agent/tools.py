"""Tools of the agent runtime (agent/registry.go:11-104, agent/tools/bash.go, file.go, skill.go).

A tool is a name, a description, a JSON schema of its arguments and a function from (arguments, working directory) to text;
tools that change things say so (``needs_approval``) and name the scope an "always allow" answer covers: the exact command
for the shell, the tool as a whole for the file writers.  File paths are resolved against the session's working directory,
which the shell tool moves when a command ends in another directory.
"""
from __future__ import annotations

import os
import subprocess
import tempfile
from dataclasses import dataclass, field
from typing import Any, Callable

BASH_TIMEOUT = 120.0
READ_LIMIT_LINES = 2000


class ToolError(Exception):
    pass


@dataclass
class ToolResult:
    content: str
    working_dir: str = ""          # non-empty: the session moves here


@dataclass
class Tool:
    name: str
    description: str
    parameters: dict[str, Any]
    run: Callable[[dict[str, Any], str], ToolResult]
    needs_approval: bool = False
    scope: Callable[[dict[str, Any]], str] | None = None

    def schema(self) -> dict[str, Any]:
        return {"type": "function", "function": {"name": self.name, "description": self.description, "parameters": self.parameters}}

    def approval_scope(self, args: dict[str, Any]) -> str:
        return self.scope(args) if self.scope else self.name


@dataclass
class Registry:
    tools: dict[str, Tool] = field(default_factory=dict)

    def register(self, tool: Tool) -> None:
        self.tools[tool.name] = tool

    def names(self) -> list[str]:
        return sorted(self.tools)

    def schemas(self) -> list[dict[str, Any]]:
        return [self.tools[n].schema() for n in self.names()]

    def execute(self, name: str, args: dict[str, Any], cwd: str) -> ToolResult:
        tool = self.tools.get(name)
        if tool is None:
            raise ToolError(f"unknown tool: {name}")
        return tool.run(args or {}, cwd)


def _string(args: dict[str, Any], key: str, required: bool = True) -> str:
    v = args.get(key)
    if v is None and not required:
        return ""
    if not isinstance(v, str) or (required and not v.strip()):
        raise ToolError(f"{key} parameter is required")
    return v


def _resolve(path: str, cwd: str) -> str:
    return os.path.normpath(path if os.path.isabs(path) else os.path.join(cwd, os.path.expanduser(path)))


# -- shell ----------------------------------------------------------------------------------------------
def _bash(args: dict[str, Any], cwd: str) -> ToolResult:
    """Runs the command in a shell of its own, bounded in time; the directory the shell ends in becomes the session's."""
    command = _string(args, "command")
    if "\x00" in command:
        raise ToolError("command contains a NUL byte")
    with tempfile.NamedTemporaryFile("r", prefix="agent-cwd-", delete=True) as marker:
        script = f"{command}\n__rc=$?\npwd > {marker.name!r} 2>/dev/null\nexit $__rc"
        try:
            p = subprocess.run(["bash", "-c", script], cwd=cwd or None, capture_output=True, text=True, timeout=BASH_TIMEOUT, stdin=subprocess.DEVNULL,
                               errors="replace")
        except subprocess.TimeoutExpired as e:
            out = (e.stdout or b"").decode(errors="replace") if isinstance(e.stdout, bytes) else (e.stdout or "")
            return ToolResult(out + f"\n[command timed out after {int(BASH_TIMEOUT)} s]")
        except OSError as e:
            raise ToolError(f"could not start the shell: {e}") from None
        new_cwd = marker.read().strip()
    text = p.stdout
    if p.stderr:
        text += ("\n" if text and not text.endswith("\n") else "") + p.stderr
    if p.returncode != 0:
        text += ("\n" if text and not text.endswith("\n") else "") + f"[exit code {p.returncode}]"
    return ToolResult(text or "(no output)", new_cwd if new_cwd and os.path.isdir(new_cwd) and new_cwd != cwd else "")


# -- files ----------------------------------------------------------------------------------------------
def _read_file(args: dict[str, Any], cwd: str) -> ToolResult:
    path = _resolve(_string(args, "path"), cwd)
    offset, limit = int(args.get("offset") or 1), int(args.get("limit") or READ_LIMIT_LINES)
    if offset < 1 or limit < 1:
        raise ToolError("offset and limit must be positive")
    try:
        with open(path, encoding="utf-8", errors="replace") as f:
            lines = f.read().splitlines()
    except IsADirectoryError:
        raise ToolError(f"{path} is a directory; use list_dir") from None
    except OSError as e:
        raise ToolError(f"cannot read {path}: {e.strerror or e}") from None
    chunk = lines[offset - 1:offset - 1 + limit]
    body = "\n".join(f"{offset + i:6d}\t{ln}" for i, ln in enumerate(chunk))
    rest = len(lines) - (offset - 1 + len(chunk))
    return ToolResult(body + (f"\n[{rest} more lines; continue with offset={offset + len(chunk)}]" if rest > 0 else "") if chunk else "(empty)")


def _write_file(args: dict[str, Any], cwd: str) -> ToolResult:
    path = _resolve(_string(args, "path"), cwd)
    content = args.get("content")
    if not isinstance(content, str):
        raise ToolError("content parameter is required")
    try:
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(path, "w", encoding="utf-8") as f:
            f.write(content)
    except OSError as e:
        raise ToolError(f"cannot write {path}: {e.strerror or e}") from None
    return ToolResult(f"wrote {len(content.encode())} bytes to {path}")


def _edit_file(args: dict[str, Any], cwd: str) -> ToolResult:
    """Replaces one exact occurrence (or every one with ``replace_all``); an ambiguous or missing match changes nothing."""
    path = _resolve(_string(args, "path"), cwd)
    old, new = args.get("old_string"), args.get("new_string")
    if not isinstance(old, str) or not isinstance(new, str) or old == "":
        raise ToolError("old_string and new_string parameters are required")
    if old == new:
        raise ToolError("old_string and new_string are the same")
    try:
        with open(path, encoding="utf-8") as f:
            text = f.read()
    except OSError as e:
        raise ToolError(f"cannot read {path}: {e.strerror or e}") from None
    n = text.count(old)
    if n == 0:
        raise ToolError("old_string was not found in the file")
    if n > 1 and not args.get("replace_all"):
        raise ToolError(f"old_string occurs {n} times; give more context or set replace_all")
    with open(path, "w", encoding="utf-8") as f:
        f.write(text.replace(old, new) if args.get("replace_all") else text.replace(old, new, 1))
    return ToolResult(f"replaced {n if args.get('replace_all') else 1} occurrence(s) in {path}")


def _list_dir(args: dict[str, Any], cwd: str) -> ToolResult:
    path = _resolve(_string(args, "path", required=False) or ".", cwd)
    try:
        names = sorted(os.listdir(path))
    except OSError as e:
        raise ToolError(f"cannot list {path}: {e.strerror or e}") from None
    return ToolResult("\n".join(n + ("/" if os.path.isdir(os.path.join(path, n)) else "") for n in names) or "(empty)")


def _obj(props: dict[str, Any], required: list[str]) -> dict[str, Any]:
    return {"type": "object", "required": required, "properties": props}


def default_registry(skills=None) -> Registry:
    r = Registry()
    s = lambda d: {"type": "string", "description": d}      # noqa: E731
    r.register(Tool("bash", "Run a shell command in the working directory and return its output.",
                    _obj({"command": s("The command line to run with bash")}, ["command"]), _bash, needs_approval=True,
                    scope=lambda a: "bash\x00" + a["command"].strip() if isinstance(a.get("command"), str) and a["command"].strip() else "bash"))
    r.register(Tool("read_file", "Read a text file with line numbers.",
                    _obj({"path": s("File to read"), "offset": {"type": "integer", "description": "First line (1-based)"},
                          "limit": {"type": "integer", "description": "Number of lines"}}, ["path"]), _read_file))
    r.register(Tool("write_file", "Create or overwrite a file.", _obj({"path": s("File to write"), "content": s("Full content")}, ["path", "content"]),
                    _write_file, needs_approval=True))
    r.register(Tool("edit_file", "Replace an exact piece of text in a file.",
                    _obj({"path": s("File to change"), "old_string": s("Text to replace (must match exactly)"), "new_string": s("Replacement"),
                          "replace_all": {"type": "boolean", "description": "Replace every occurrence"}}, ["path", "old_string", "new_string"]),
                    _edit_file, needs_approval=True))
    r.register(Tool("list_dir", "List a directory.", _obj({"path": s("Directory (default: working directory)")}, []), _list_dir))
    if skills is not None and skills.names():
        r.register(Tool("skill", "Load the instructions of a named skill: " + ", ".join(skills.names()) + ".",
                        _obj({"name": s("Skill to load")}, ["name"]), lambda a, cwd: ToolResult(skills.load(_string(a, "name")))))
    return r
