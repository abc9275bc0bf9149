"""Skills: folders with a ``SKILL.md`` whose front matter names and describes them (agent/skills.go:30-200).

A skill is loaded on demand, by the model through the ``skill`` tool or by the caller for a whole run; its body then
enters the conversation as the result of a synthetic tool call, so that it is part of the history like any tool output.
"""
from __future__ import annotations

import os
import re

_FRONT = re.compile(r"\A---\s*\n(.*?)\n---\s*\n?(.*)\Z", re.S)


class SkillCatalog:
    def __init__(self, roots: list[str] | None = None):
        home = os.path.expanduser("~")
        self.roots = roots if roots is not None else [os.path.join(home, ".ollama", "skills"), os.path.join(os.getcwd(), ".ollama", "skills")]
        self.skills: dict[str, tuple[str, str]] = {}          # name -> (description, path of SKILL.md)
        for root in self.roots:
            try:
                entries = sorted(os.listdir(root))
            except OSError:
                continue
            for d in entries:
                path = os.path.join(root, d, "SKILL.md")
                meta = self._meta(path)
                if meta is not None:
                    self.skills[meta[0] or d] = (meta[1], path)      # a later root overrides an earlier one

    @staticmethod
    def _meta(path: str) -> tuple[str, str] | None:
        try:
            with open(path, encoding="utf-8") as f:
                m = _FRONT.match(f.read(65536))
        except OSError:
            return None
        if m is None:
            return ("", "")
        fields = dict((k.strip(), v.strip().strip("\"'")) for k, _, v in (ln.partition(":") for ln in m.group(1).splitlines()) if _)
        return fields.get("name", ""), fields.get("description", "")

    def names(self) -> list[str]:
        return sorted(self.skills)

    def describe(self) -> str:
        return "\n".join(f"- {n}: {self.skills[n][0]}" for n in self.names())

    def load(self, name: str) -> str:
        if name not in self.skills:
            raise KeyError(f"unknown skill: {name} (available: {', '.join(self.names()) or 'none'})")
        with open(self.skills[name][1], encoding="utf-8") as f:
            text = f.read()
        m = _FRONT.match(text)
        base = os.path.dirname(self.skills[name][1])
        return f"Skill {name} (files in {base}):\n\n" + (m.group(2) if m else text).strip()
