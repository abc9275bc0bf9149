"""``launch``: start a third-party coding tool wired to this server.

The reference ships a registry of integrations (cmd/launch/registry.go:36-325), each knowing how to find its tool, how to
point it at the local server (environment, command-line overrides, or an edit of the tool's own settings file) and which
model list to offer, a saved choice per integration in ``~/.ollama/config.json`` (cmd/config/config.go:13-30) and terminal
pickers for the integration and the model.  Here an integration is a row of data plus, where a tool needs more than
environment and arguments, one small function that edits its settings; the set covers the tools whose wiring is fully
described by the reference's own sources: Claude Code (claude.go:63-83, 172-180), Codex (codex.go:35-49, 174-185),
OpenCode (opencode.go:289-315, 346-386) and Droid (droid.go:67-150).  Settings files are rewritten atomically with a
``.bak`` copy of the previous content next to them.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Any, Callable

from .. import envconfig
from . import tui


@dataclass
class LaunchModel:
    name: str
    capabilities: list[str] = field(default_factory=list)
    context_length: int = 0
    max_output_tokens: int = 0


def host_url() -> str:
    """Where a local tool reaches the server: the configured address, with "every interface" read as this machine."""
    h = envconfig.host()
    name = "127.0.0.1" if h.host in ("", "0.0.0.0", "::") else h.host
    return f"{h.scheme}://{'[' + name + ']' if ':' in name else name}:{h.port}"


# -- per-tool wiring ---------------------------------------------------------------------------------
def claude_env(model: str, models: list[LaunchModel]) -> dict[str, str]:
    env = {"ANTHROPIC_BASE_URL": host_url(), "ANTHROPIC_API_KEY": "", "ANTHROPIC_AUTH_TOKEN": "ollama", "CLAUDE_CODE_ATTRIBUTION_HEADER": "0",
           "CLAUDE_CODE_TOTAL_TOKENS_REMINDER": "off", "DISABLE_ERROR_REPORTING": "1", "DISABLE_FEEDBACK_COMMAND": "1",
           "CLAUDE_CODE_DISABLE_FEEDBACK_SURVEY": "1"}
    for key in ("ANTHROPIC_DEFAULT_OPUS_MODEL", "ANTHROPIC_DEFAULT_SONNET_MODEL", "ANTHROPIC_DEFAULT_HAIKU_MODEL", "CLAUDE_CODE_SUBAGENT_MODEL"):
        env[key] = model
    return env


CODEX_PROFILE = "ollama-launch"


def codex_args(model: str, extra: list[str]) -> list[str]:
    for a in extra:          # the launcher owns the provider wiring: overrides that would undo it are refused
        key = a.split("=", 1)[0].strip().strip("\"'")
        if "=" in a and (key in ("profile", "model", "model_provider", "model_catalog_json") or key.startswith("model_providers.")):
            raise LaunchError(f"codex: the option {a!r} conflicts with the launch configuration")
    base = host_url() + "/v1/"
    over = [f'model_provider="{CODEX_PROFILE}"', f'model_providers.{CODEX_PROFILE}.name="Ollama"', f'model_providers.{CODEX_PROFILE}.base_url="{base}"',
            f'model_providers.{CODEX_PROFILE}.wire_api="responses"']
    args: list[str] = []
    for o in over:
        args += ["-c", o]
    return args + (["-m", model] if model else []) + extra


def opencode_env(model: str, models: list[LaunchModel]) -> dict[str, str]:
    entries: dict[str, Any] = {}
    for m in models or [LaunchModel(model)]:
        e: dict[str, Any] = {"name": m.name}
        if "vision" in m.capabilities:
            e["modalities"] = {"input": ["text", "image"], "output": ["text"]}
        if "thinking" in m.capabilities:
            e["reasoning"] = True
            e["variants"] = {"none": {"reasoningEffort": "none"}, "low": {"disabled": True}, "medium": {"disabled": True}, "high": {"disabled": True}}
        if m.max_output_tokens > 0:
            e["limit"] = {**({"context": m.context_length} if m.context_length > 0 else {}), "output": m.max_output_tokens}
        entries[m.name] = e
    cfg = {"$schema": "https://opencode.ai/config.json", "model": "ollama/" + model,
           "provider": {"ollama": {"npm": "@ai-sdk/openai-compatible", "name": "Ollama", "options": {"baseURL": host_url() + "/v1"}, "models": entries}}}
    return {"OPENCODE_CONFIG_CONTENT": json.dumps(cfg, separators=(",", ":"))}


def write_with_backup(path: str, text: str) -> None:
    os.makedirs(os.path.dirname(path), exist_ok=True)
    if os.path.exists(path):
        shutil.copy2(path, path + ".bak")
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        f.write(text)
    os.replace(tmp, path)


def droid_configure(model: str, models: list[LaunchModel], home: str | None = None) -> str:
    """``~/.factory/settings.json``: our models replace the entries of an earlier launch (recognised by their api key) in front of
    the user's own custom models; the first becomes the session default."""
    path = os.path.join(home or os.path.expanduser("~"), ".factory", "settings.json")
    settings: dict[str, Any] = {}
    if os.path.exists(path):
        try:
            with open(path, encoding="utf-8") as f:
                settings = json.load(f)
        except ValueError as e:
            raise LaunchError(f"failed to parse settings file: {e}, at: {path}") from None
        if not isinstance(settings, dict):
            raise LaunchError(f"failed to parse settings file: not an object, at: {path}")
    theirs = [m for m in settings.get("customModels") or [] if isinstance(m, dict) and m.get("apiKey") != "ollama"]
    ours = [{"model": m.name, "displayName": m.name, "baseUrl": host_url() + "/v1", "apiKey": "ollama", "provider": "generic-chat-completion-api",
             "maxOutputTokens": m.max_output_tokens or 64000, "supportsImages": "vision" in m.capabilities, "id": f"custom:{m.name}-{i}", "index": i}
            for i, m in enumerate(models or [LaunchModel(model)])]
    settings["customModels"] = ours + theirs
    session = settings.get("sessionDefaultSettings") if isinstance(settings.get("sessionDefaultSettings"), dict) else {}
    session["model"] = ours[0]["id"]
    if session.get("reasoningEffort") not in ("high", "medium", "low", "none"):
        session["reasoningEffort"] = "none"
    settings["sessionDefaultSettings"] = session
    write_with_backup(path, json.dumps(settings, indent=2))
    return path


class LaunchError(Exception):
    pass


@dataclass
class Integration:
    name: str
    display: str
    description: str
    binary: str
    aliases: tuple[str, ...] = ()
    install_url: str = ""
    install_command: tuple[str, ...] = ()
    env: Callable[[str, list[LaunchModel]], dict[str, str]] | None = None
    args: Callable[[str, list[str]], list[str]] | None = None
    configure: Callable[[str, list[LaunchModel]], str] | None = None
    fallback_paths: tuple[str, ...] = ()
    hidden: bool = False

    def find(self) -> str | None:
        p = shutil.which(self.binary)
        if p:
            return p
        home = os.path.expanduser("~")
        return next((q for q in (os.path.join(home, f) for f in self.fallback_paths) if os.path.exists(q)), None)

    def install_hint(self) -> str:
        how = []
        if self.install_command:
            how.append("  " + " ".join(self.install_command))
        if self.install_url:
            how.append("  " + self.install_url)
        return f"{self.display} is not installed." + ("\n\nInstall it with:\n" + "\n".join(how) if how else "") + f"\n\nThen re-run:\n  ollama launch {self.name}"


INTEGRATIONS = [
    Integration("claude", "Claude Code", "Anthropic's coding tool with subagents", "claude", install_url="https://code.claude.com/docs/en/quickstart",
                env=claude_env, args=lambda model, extra: (["--model", model] if model else []) + extra,
                fallback_paths=(".local/bin/claude", ".claude/local/claude")),
    Integration("opencode", "OpenCode", "Anomaly's open-source coding agent", "opencode", install_url="https://opencode.ai", env=opencode_env,
                args=lambda model, extra: list(extra), fallback_paths=(".opencode/bin/opencode",)),
    Integration("codex", "Codex", "OpenAI's open-source coding agent", "codex", install_url="https://developers.openai.com/codex/cli/",
                install_command=("npm", "install", "-g", "@openai/codex"), env=lambda model, models: {"OPENAI_API_KEY": "ollama"}, args=codex_args),
    Integration("droid", "Droid", "Factory's coding agent across terminal and IDEs", "droid", install_url="https://docs.factory.ai/cli/getting-started/quickstart",
                args=lambda model, extra: list(extra), configure=droid_configure),
]
ORDER = ["claude", "opencode", "codex", "droid"]


def lookup(name: str) -> Integration:
    key = name.strip().lower()
    for it in INTEGRATIONS:
        if key == it.name or key in it.aliases:
            return it
    raise LaunchError(f"unknown integration: {name}")


# -- saved choices ---------------------------------------------------------------------------------------
def config_path() -> str:
    return os.path.join(os.path.expanduser("~"), ".ollama", "config.json")


def load_config() -> dict[str, Any]:
    try:
        with open(config_path(), encoding="utf-8") as f:
            cfg = json.load(f)
        return cfg if isinstance(cfg, dict) else {}
    except (OSError, ValueError):
        return {}


def save_choice(integration: str, models: list[str]) -> None:
    cfg = load_config()
    table = cfg.setdefault("integrations", {})
    entry = table.get(integration) if isinstance(table.get(integration), dict) else {}
    entry["models"] = models
    table[integration] = entry
    cfg["last_selection"] = integration
    if models:
        cfg["last_model"] = models[0]
    write_with_backup(config_path(), json.dumps(cfg, indent=2))


def saved_models(integration: str) -> list[str]:
    entry = (load_config().get("integrations") or {}).get(integration)
    return [m for m in (entry or {}).get("models") or [] if isinstance(m, str)]


# -- the command ------------------------------------------------------------------------------------------
def available_models(client) -> list[LaunchModel]:
    out = []
    for m in client.list().get("models", []):
        caps, ctx = [], 0
        try:
            info = client.show(m["name"])
            caps = list(info.get("capabilities") or [])
            ctx = next((int(v) for k, v in (info.get("model_info") or {}).items() if k.endswith(".context_length")), 0)
        except Exception:
            pass
        out.append(LaunchModel(m["name"], caps, ctx))
    return out


def plan(it: Integration, model: str, models: list[LaunchModel], extra: list[str]) -> tuple[list[str], dict[str, str]]:
    """Command line and environment additions for one launch (no side effects: what ``--dry-run`` prints)."""
    binary = it.find() or it.binary
    args = it.args(model, extra) if it.args else list(extra)
    env = it.env(model, models) if it.env else {}
    return [binary] + args, env


def launch(client, name: str | None, model: str | None, extra: list[str], choose_only: bool = False, dry_run: bool = False,
           run: Callable[..., int] | None = None, inp=None, out=None) -> int:
    out = out or sys.stderr
    try:
        if not name:
            items = [tui.Item(i.name, i.description) for i in sorted((i for i in INTEGRATIONS if not i.hidden), key=lambda i: ORDER.index(i.name))]
            name = tui.select("Select an integration:", items, inp, out)
        it = lookup(name)
        models = available_models(client)
        if not model:
            saved = [m for m in saved_models(it.name) if any(m == x.name for x in models)]
            if saved and not choose_only:
                model = saved[0]
            else:
                if not models:
                    raise LaunchError("no models are installed; pull one first (ollama pull <model>)")
                tools = [m for m in models if "tools" in m.capabilities] or models      # coding tools need tool calling
                model = tui.select(f"Select a model for {it.display}:", [tui.Item(m.name, ", ".join(m.capabilities)) for m in tools], inp, out)
        elif not any(model == m.name or model + ":latest" == m.name for m in models):
            raise LaunchError(f"model '{model}' not found; pull it first (ollama pull {model})")
        chosen = [m for m in models if m.name in (model, model + ":latest")] + [m for m in models if m.name not in (model, model + ":latest")]
        save_choice(it.name, [model])
        if choose_only:
            out.write(f"{it.display} will use {model}\n")
            return 0
        if it.find() is None and not dry_run:
            raise LaunchError(it.install_hint())
        if it.configure and not dry_run:
            path = it.configure(model, chosen)
            out.write(f"updated {path}\n")
        cmd, env = plan(it, model, chosen, extra)
        if dry_run:
            out.write(" ".join(f"{k}={v}" for k, v in env.items() if k != "OPENCODE_CONFIG_CONTENT") + (" " if env else "") + " ".join(cmd) + "\n")
            return 0
        out.write(f"Launching {it.display} with {model}...\n")
        return (run or subprocess.call)(cmd, env={**os.environ, **env})
    except tui.Cancelled as e:
        out.write(f"{e}\n")
        return 130
    except LaunchError as e:
        out.write(f"Error: {e}\n")
        return 1
