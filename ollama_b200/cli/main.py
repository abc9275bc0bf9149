"""Command line: ``python -m ollama_b200 <command>``.

Every command except ``serve`` (and the worker entry points) is a thin client of the REST API, as in the
reference (cmd/cmd.go:2279-2555: serve, create, show, run, stop, pull, push, list, ps, cp, rm; the REPL of
``run`` with its /set, /show, /clear, /bye commands is cmd/interactive.go).  ``bench`` reproduces the
reference's standalone benchmark tool (cmd/bench/bench.go): warm-up, epochs, TTFT from the first streamed
chunk, prefill / generate rates from the API's own counters.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import re
import sys
import time
from typing import Any

from .. import envconfig
from ..api.client import Client, ResponseError
from ..utils.format import human_ago, human_bytes
from ..version import VERSION


# ---------------------------------------------------------------------------------------------------
# formatting helpers
# ---------------------------------------------------------------------------------------------------
def table(rows: list[list[str]], header: list[str]) -> str:
    cols = [header] + rows
    widths = [max(len(r[i]) for r in cols) for i in range(len(header))]
    return "\n".join("    ".join(c.ljust(w) for c, w in zip(r, widths)).rstrip() for r in cols)


def progress_line(ev: dict[str, Any], last: dict[str, Any]) -> None:
    """One status line per event; layer transfers are rewritten in place with a percentage."""
    status = ev.get("status", "")
    if ev.get("total"):
        pct = 100.0 * ev.get("completed", 0) / max(ev["total"], 1)
        sys.stderr.write(f"\r{status}: {pct:5.1f}% of {human_bytes(ev['total'])}   ")
        last["inline"] = True
    else:
        if last.get("inline"):
            sys.stderr.write("\n")
            last["inline"] = False
        if status != last.get("status"):
            sys.stderr.write(status + "\n")
    last["status"] = status
    sys.stderr.flush()


# ---------------------------------------------------------------------------------------------------
# commands
# ---------------------------------------------------------------------------------------------------
def cmd_serve(args) -> int:
    import uvicorn
    from ..server.routes import create_app
    from ..utils import logutil
    logutil.setup()
    try:      # the installation's identity for registry pushes and private pulls (cmd/cmd.go:2015-2077)
        from .. import auth
        auth.ensure_key()
    except (auth.AuthError, OSError) as e:
        print(f"warning: could not set up the ed25519 key pair: {e}", file=sys.stderr)
    try:      # start-up housekeeping of the blob store (server/routes.go Serve: fixBlobs, then PruneLayers unless OLLAMA_NOPRUNE)
        from ..store import manifest
        if os.path.isdir(manifest.blobs_dir()):
            manifest.fix_blobs()
            if not envconfig.no_prune():
                manifest.prune_layers()
                manifest.prune_empty_dirs(manifest.manifests_dir())
    except OSError as e:
        print(f"warning: could not tidy the model store: {e}", file=sys.stderr)
    h = envconfig.host()
    print(f"ollama-b200 {VERSION} listening on {h.netloc}", file=sys.stderr)
    for k, (v, desc) in envconfig.as_map().items():
        print(f"  {k}={v}", file=sys.stderr)
    uvicorn.run(create_app(), host=h.host or "0.0.0.0", port=h.port, log_level="info" if envconfig.log_level() <= 20 else "warning")
    return 0


def cmd_list(args) -> int:
    models = Client().list().get("models", [])
    rows = [[m["name"], m.get("digest", "")[:12], human_bytes(m.get("size", 0)), human_ago(m.get("modified_at", ""))] for m in models]
    print(table(rows, ["NAME", "ID", "SIZE", "MODIFIED"]))
    return 0


def cmd_ps(args) -> int:
    rows = []
    for m in Client().ps().get("models", []):
        size, vram = m.get("size", 0), m.get("size_vram", 0)
        if vram >= size or size == 0:
            proc = "100% GPU"
        elif vram == 0:
            proc = "100% CPU"
        else:
            g = round(100 * vram / size)
            proc = f"{100 - g}%/{g}% CPU/GPU"
        rows.append([m["name"], m.get("digest", "")[:12], human_bytes(size), proc, str(m.get("context_length", "")), human_ago(m.get("expires_at", ""))])
    print(table(rows, ["NAME", "ID", "SIZE", "PROCESSOR", "CONTEXT", "UNTIL"]))
    return 0


def cmd_show(args) -> int:
    info = Client().show(args.model, verbose=args.verbose)
    for flag in ("license", "modelfile", "parameters", "template", "system"):
        if getattr(args, flag):
            print(info.get(flag, ""))
            return 0
    d = info.get("details", {})
    mi = info.get("model_info", {})
    arch = mi.get("general.architecture", d.get("family", ""))
    print("  Model")
    for k, v in (("architecture", arch), ("parameters", d.get("parameter_size", "")), ("context length", mi.get(f"{arch}.context_length", "")),
                 ("embedding length", mi.get(f"{arch}.embedding_length", "")), ("quantization", d.get("quantization_level", ""))):
        if v != "":
            print(f"    {k:<20}{v}")
    if info.get("capabilities"):
        print("\n  Capabilities")
        for c in info["capabilities"]:
            print(f"    {c}")
    if info.get("parameters"):
        print("\n  Parameters")
        for line in info["parameters"].splitlines():
            print(f"    {line}")
    if info.get("system"):
        print("\n  System\n    " + info["system"].replace("\n", "\n    "))
    if info.get("license"):
        print("\n  License\n    " + "\n    ".join(info["license"].splitlines()[:2]))
    return 0


def cmd_cp(args) -> int:
    Client().copy(args.source, args.destination)
    print(f"copied '{args.source}' to '{args.destination}'")
    return 0


def cmd_rm(args) -> int:
    c = Client()
    for m in args.models:
        c.delete(m)
        print(f"deleted '{m}'")
    return 0


def cmd_stop(args) -> int:
    for _ in Client().generate(model=args.model, keep_alive=0, stream=False):
        pass
    return 0


def cmd_pull(args) -> int:
    last: dict[str, Any] = {}
    for ev in Client().pull(args.model, insecure=args.insecure):
        progress_line(ev, last)
    sys.stderr.write("\n" if last.get("inline") else "")
    return 0


def cmd_push(args) -> int:
    last: dict[str, Any] = {}
    for ev in Client().push(args.model, insecure=args.insecure):
        progress_line(ev, last)
    sys.stderr.write("\n" if last.get("inline") else "")
    return 0


def _upload(c: Client, path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    digest = "sha256:" + h.hexdigest()
    if not c.blob_exists(digest):
        with open(path, "rb") as f:
            c.create_blob(digest, f.read())
    return digest


def cmd_create(args) -> int:
    from ..store.modelfile import parse_modelfile
    path = args.file or "Modelfile"
    with open(path, "rb") as f:
        mf = parse_modelfile(f.read())
    req = mf.create_request()
    req["model"] = args.model
    if args.quantize:
        req["quantize"] = args.quantize
    c = Client()
    base = os.path.dirname(os.path.abspath(path))

    def local(p: str) -> str | None:
        q = os.path.expanduser(p)
        q = q if os.path.isabs(q) else os.path.join(base, q)
        return q if os.path.exists(q) else None

    src = req.get("from", "")
    lp = local(src) if src else None
    if lp:       # a GGUF file or a directory of weights on this machine: upload as blobs, reference by digest
        files = {}
        paths = [lp] if os.path.isfile(lp) else [os.path.join(lp, n) for n in sorted(os.listdir(lp)) if os.path.isfile(os.path.join(lp, n))]
        for p in paths:
            print(f"copying file {os.path.basename(p)}", file=sys.stderr)
            files[os.path.basename(p)] = _upload(c, p)
        req.pop("from")
        req["files"] = files
    for key in ("adapter_paths", "draft_paths"):
        for p in req.pop(key, []):
            lp2 = local(p)
            if not lp2:
                raise SystemExit(f"Error: {p}: no such file")
            if key == "draft_paths" and lp and os.path.realpath(lp2) == os.path.realpath(lp):
                raise SystemExit("Error: DRAFT must not reference the same local path as FROM")
            req.setdefault("adapters" if key == "adapter_paths" else "draft_files", {})[os.path.basename(lp2)] = _upload(c, lp2)
    last: dict[str, Any] = {}
    for ev in c.create(**req):
        progress_line(ev, last)
    return 0


_MEDIA_PATH = re.compile(r"(?:[a-zA-Z]:)?(?:\./|/|\\)[\S\\ ]+?\.(?i:jpg|jpeg|png|webp|wav)\b")
_MEDIA_MAGIC = ((b"\xff\xd8\xff", "image/jpeg"), (b"\x89PNG\r\n\x1a\n", "image/png"), (b"RIFF", "riff"))
_UNESCAPE = {"\\ ": " ", "\\(": "(", "\\)": ")", "\\[": "[", "\\]": "]", "\\{": "{", "\\}": "}", "\\$": "$", "\\&": "&", "\\;": ";",
             "\\'": "'", "\\\\": "\\", "\\*": "*", "\\?": "?", "\\~": "~", "%20": " "}


def _media_type(head: bytes) -> str:
    for magic, kind in _MEDIA_MAGIC:
        if head.startswith(magic):
            if kind == "riff":
                return {b"WEBP": "image/webp", b"WAVE": "audio/wave"}.get(head[8:12], "")
            return kind
    return ""


def extract_media(text: str) -> tuple[str, list[str]]:
    """File paths of images (or audio) inside a prompt -> (prompt without them, their contents as base64), as the reference's
    prompt line does (cmd/interactive.go:605-644, :700-740): a path starts with ``/``, ``./``, a backslash or a drive letter,
    may contain escaped spaces, and ends in jpg / jpeg / png / webp / wav; strings that name no existing file stay in the text;
    a file that exists must really be one of those types and at most 100 MB."""
    import base64
    images: list[str] = []
    for found in _MEDIA_PATH.findall(text):
        path = found
        for a, b in _UNESCAPE.items():
            path = path.replace(a, b)
        try:
            with open(path, "rb") as f:
                data = f.read(100 * 1024 * 1024 + 1)
        except FileNotFoundError:
            continue
        except OSError as e:
            raise ValueError(f"couldn't process file: {e}")
        if len(data) > 100 * 1024 * 1024:
            raise ValueError("file size exceeds maximum limit (100MB)")
        kind = _media_type(data[:512])
        if not kind:
            raise ValueError(f"invalid file type: {path}")
        print(f"Added {'audio' if kind.startswith('audio') else 'image'} '{path}'", file=sys.stderr)
        for quoted in ("'" + path + "'", "'" + found + "'", found):
            text = text.replace(quoted, "")
        images.append(base64.b64encode(data).decode())
    return text.strip(), images


class Repl:
    """Interactive chat session of ``run`` (cmd/interactive.go in the reference)."""

    HELP = ("Available Commands:\n  /set            Set session variables\n  /show           Show model information\n"
            "  /load <model>   Load a session or model\n  /save <model>   Save your current session\n"
            "  /clear          Clear session context\n  /bye            Exit\n  /?, /help       Help for a command\n\n"
            'Use """ to begin a multi-line message.\n')

    def __init__(self, client: Client, model: str, opts: dict[str, Any], fmt: str, think: Any, keep_alive: Any, verbose: bool):
        self.c, self.model, self.opts, self.fmt, self.think, self.keep_alive, self.verbose = client, model, opts, fmt, think, keep_alive, verbose
        self.messages: list[dict[str, Any]] = []
        self.system = ""

    def turn(self, text: str) -> None:
        try:
            text, images = extract_media(text)
        except ValueError as e:
            print(f"Error: {e}", file=sys.stderr)
            return
        self.messages.append({"role": "user", "content": text, **({"images": images} if images else {})})
        req: dict[str, Any] = {"model": self.model, "messages": ([{"role": "system", "content": self.system}] if self.system else []) + self.messages,
                               "options": self.opts}
        if self.fmt:
            req["format"] = self.fmt
        if self.think is not None:
            req["think"] = self.think
        if self.keep_alive is not None:
            req["keep_alive"] = self.keep_alive
        answer, thinking_open, final = [], False, {}
        for ev in self.c.chat(**req):
            msg = ev.get("message", {})
            if msg.get("thinking"):
                if not thinking_open:
                    sys.stdout.write("Thinking...\n")
                    thinking_open = True
                sys.stdout.write(msg["thinking"])
            if msg.get("content"):
                if thinking_open:
                    sys.stdout.write("\n...done thinking.\n\n")
                    thinking_open = False
                sys.stdout.write(msg["content"])
                answer.append(msg["content"])
            for tc in msg.get("tool_calls") or []:
                sys.stdout.write(f"\n[tool call] {json.dumps(tc.get('function', {}))}\n")
            sys.stdout.flush()
            if ev.get("done"):
                final = ev
        sys.stdout.write("\n\n")
        self.messages.append({"role": "assistant", "content": "".join(answer)})
        if self.verbose:
            print_metrics(final)

    def command(self, line: str) -> bool:
        parts = line.split()
        if parts[0] in ("/bye", "/exit"):
            return False
        if parts[0] in ("/?", "/help"):
            print(self.HELP)
        elif parts[0] == "/clear":
            self.messages.clear()
            print("Cleared session context")
        elif parts[0] == "/load":
            if len(parts) != 2:
                print("Usage:\n  /load <modelname>")
                return True
            try:                                    # a new model starts a new conversation (cmd/interactive.go:209-252)
                self.c.show(parts[1])
            except Exception as e:
                print(f"Couldn't find model '{parts[1]}'" if "not found" in str(e) else f"error: {e}")
                return True
            print(f"Loading model '{parts[1]}'")
            self.model, self.messages = parts[1], []
            for _ in self.c.generate(model=self.model, prompt="", keep_alive=self.keep_alive):
                pass
        elif parts[0] == "/save":
            if len(parts) != 2:
                print("Usage:\n  /save <modelname>")
                return True
            req: dict[str, Any] = {"model": parts[1], "from": self.model, "messages": list(self.messages)}
            if self.system:
                req["system"] = self.system
            if self.opts:
                req["parameters"] = dict(self.opts)
            try:                                    # the session becomes a model: system text, parameters and the conversation so far
                for _ in self.c.create(**req):
                    pass
                print(f"Created new model '{parts[1]}'")
            except Exception as e:
                print(f"error: The model name '{parts[1]}' is invalid" if "invalid model name" in str(e) else f"error: {e}")
        elif parts[0] == "/show":
            info = self.c.show(self.model)
            what = parts[1] if len(parts) > 1 else "info"
            print(info.get(what, "") if what != "info" else json.dumps(info.get("details", {}), indent=2))
        elif parts[0] == "/set" and len(parts) >= 2:
            if parts[1] == "parameter" and len(parts) >= 4:
                v: Any = " ".join(parts[3:])
                try:
                    v = json.loads(v)
                except ValueError:
                    pass
                self.opts[parts[2]] = v
                print(f"Set parameter '{parts[2]}' to '{v}'")
            elif parts[1] == "system":
                self.system = line.split(None, 2)[2].strip('"') if len(parts) > 2 else ""
                print("Set system message.")
            elif parts[1] in ("verbose", "quiet"):
                self.verbose = parts[1] == "verbose"
            elif parts[1] in ("history", "nohistory"):
                if getattr(self, "editor", None) is not None:
                    self.editor.set_enabled(parts[1] == "history")
                print("Enabled history." if parts[1] == "history" else "Disabled history.")
            elif parts[1] in ("think", "nothink"):
                self.think = parts[1] == "think" if len(parts) < 3 else parts[2]
            elif parts[1] == "format" and len(parts) > 2:
                self.fmt = parts[2]
            elif parts[1] == "noformat":
                self.fmt = ""
            else:
                print(f"Unknown command '/set {parts[1]}'. Type /? for help")
        else:
            print(f"Unknown command '{parts[0]}'. Type /? for help")
        return True

    def loop(self) -> None:
        from .lineedit import LineEditor
        buf: list[str] | None = None
        self.editor = editor = LineEditor()
        while True:
            try:
                line = editor.read("... " if buf is not None else ">>> ", record=buf is None)
            except EOFError:
                print()
                return
            except KeyboardInterrupt:
                print("\nUse Ctrl + d or /bye to exit.")
                buf = None
                continue
            if buf is not None:
                if line.rstrip().endswith('"""'):
                    buf.append(line.rstrip()[:-3])
                    text, buf = "\n".join(buf), None
                    self.turn(text)
                else:
                    buf.append(line)
                continue
            if line.startswith('"""'):
                rest = line[3:]
                if rest.rstrip().endswith('"""') and len(rest.rstrip()) >= 3:
                    self.turn(rest.rstrip()[:-3])
                else:
                    buf = [rest]
                continue
            if not line.strip():
                continue
            if line.startswith("/"):
                if not self.command(line.strip()):
                    return
                continue
            try:
                self.turn(line)
            except KeyboardInterrupt:
                print()


def print_metrics(ev: dict[str, Any]) -> None:
    def sec(ns):
        return f"{ns / 1e9:.6f}s"
    rows = [("total duration", sec(ev.get("total_duration", 0))), ("load duration", sec(ev.get("load_duration", 0))),
            ("prompt eval count", f"{ev.get('prompt_eval_count', 0)} token(s)"), ("prompt eval duration", sec(ev.get("prompt_eval_duration", 0)))]
    if ev.get("prompt_eval_duration"):
        rows.append(("prompt eval rate", f"{ev.get('prompt_eval_count', 0) / (ev['prompt_eval_duration'] / 1e9):.2f} tokens/s"))
    rows += [("eval count", f"{ev.get('eval_count', 0)} token(s)"), ("eval duration", sec(ev.get("eval_duration", 0)))]
    if ev.get("eval_duration"):
        rows.append(("eval rate", f"{ev.get('eval_count', 0) / (ev['eval_duration'] / 1e9):.2f} tokens/s"))
    for k, v in rows:
        print(f"{k + ':':<22}{v}", file=sys.stderr)


def cmd_run(args) -> int:
    c = Client()
    try:
        c.show(args.model)
    except ResponseError as e:
        if e.status != 404:
            raise
        print(f"pulling '{args.model}'", file=sys.stderr)
        cmd_pull(argparse.Namespace(model=args.model, insecure=args.insecure))
    opts: dict[str, Any] = {}
    think: Any = None
    if args.think is not None:
        think = {"true": True, "false": False}.get(args.think.lower(), args.think)
    prompt = " ".join(args.prompt)
    if not sys.stdin.isatty():
        piped = sys.stdin.read()
        prompt = (prompt + "\n" + piped).strip() if prompt else piped
    if prompt:
        try:
            prompt, images = extract_media(prompt)
        except ValueError as e:
            print(f"Error: {e}", file=sys.stderr)
            return 1
        req: dict[str, Any] = {"model": args.model, "prompt": prompt, "options": opts}
        if images:
            req["images"] = images
        if args.format:
            req["format"] = args.format
        if think is not None:
            req["think"] = think
        if args.keepalive:
            req["keep_alive"] = args.keepalive
        final = {}
        for ev in c.generate(**req):
            sys.stdout.write(ev.get("response", ""))
            sys.stdout.flush()
            if ev.get("done"):
                final = ev
        sys.stdout.write("\n")
        if args.verbose:
            print_metrics(final)
        return 0
    for _ in c.generate(model=args.model, keep_alive=args.keepalive or None):      # load the model before the first prompt
        pass
    Repl(c, args.model, opts, args.format or "", think, args.keepalive or None, args.verbose).loop()
    return 0


def cmd_bench(args) -> int:
    """Epochs of one generate request per model; rates come from the server's counters, TTFT from the first streamed chunk."""
    c = Client()
    results = []
    for model in args.model.split(","):
        rng_words = ["alpha", "bravo", "charlie", "delta", "echo", "foxtrot", "golf", "hotel", "india", "juliet"]
        def prompt(epoch: int) -> str:
            if args.prompt:
                return f"[{epoch}] " + args.prompt        # vary the prefix so that no epoch reuses a cached prompt
            n = max(args.prompt_tokens, 1)
            return " ".join(rng_words[(i * 7 + epoch) % len(rng_words)] for i in range(n))
        opts = {"temperature": args.temperature, "num_predict": args.max_tokens, "seed": args.seed}
        for w in range(args.warmup):
            for _ in c.generate(model=model, prompt=prompt(-1 - w), options=opts, raw=True):
                pass
        pre, gen, ttft, load, total = [], [], [], [], []
        for e in range(args.epochs):
            t0 = time.perf_counter()
            first, final = None, {}
            for ev in c.generate(model=model, prompt=prompt(e), options=opts, raw=True, keep_alive=args.keep_alive):
                if first is None and (ev.get("response") or ev.get("thinking")):
                    first = time.perf_counter() - t0
                if ev.get("done"):
                    final = ev
            if final.get("prompt_eval_duration"):
                pre.append(final.get("prompt_eval_count", 0) / (final["prompt_eval_duration"] / 1e9))
            if final.get("eval_duration"):
                gen.append(final.get("eval_count", 0) / (final["eval_duration"] / 1e9))
            ttft.append((first or 0.0) * 1e3)
            load.append(final.get("load_duration", 0) / 1e6)
            total.append(final.get("total_duration", 0) / 1e6)
        def med(v):
            return statistics.median(v) if v else 0.0
        results.append({"model": model, "epochs": args.epochs, "prefill_tok_s": med(pre), "generate_tok_s": med(gen), "ttft_ms": med(ttft),
                        "load_ms": med(load), "total_ms": med(total)})
    if args.format == "csv":
        print("model,epochs,prefill_tok_s,generate_tok_s,ttft_ms,load_ms,total_ms")
        for r in results:
            print(",".join(str(round(v, 3)) if isinstance(v, float) else str(v) for v in r.values()))
    elif args.format == "json":
        print(json.dumps(results))
    else:       # benchstat-style lines
        for r in results:
            name = r["model"].replace(":", "_")
            if r["prefill_tok_s"]:
                print(f"BenchmarkModel/name={name}/step=prefill {r['epochs']} {1e9 / r['prefill_tok_s']:.0f} ns/token {r['prefill_tok_s']:.2f} token/sec")
            if r["generate_tok_s"]:
                print(f"BenchmarkModel/name={name}/step=generate {r['epochs']} {1e9 / r['generate_tok_s']:.0f} ns/token {r['generate_tok_s']:.2f} token/sec")
            print(f"BenchmarkModel/name={name}/step=ttft {r['epochs']} {r['ttft_ms'] * 1e6:.0f} ns/request")
            print(f"BenchmarkModel/name={name}/step=load {r['epochs']} {r['load_ms'] * 1e6:.0f} ns/request")
            print(f"BenchmarkModel/name={name}/step=total {r['epochs']} {r['total_ms'] * 1e6:.0f} ns/request")
    return 0


def cmd_gpu_discover(args) -> int:
    from ..discover.probe import main as probe_main
    return probe_main()


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="ollama-b200", description="Large language model runner for NVIDIA B200")
    ap.add_argument("-v", "--version", action="store_true", help="Show version information")
    sub = ap.add_subparsers(dest="cmd")
    sub.add_parser("serve", aliases=["start"], help="Start the server").set_defaults(fn=cmd_serve)
    p = sub.add_parser("create", help="Create a model from a Modelfile")
    p.add_argument("model")
    p.add_argument("-f", "--file", default="")
    p.add_argument("-q", "--quantize", default="")
    p.set_defaults(fn=cmd_create)
    p = sub.add_parser("show", help="Show information for a model")
    p.add_argument("model")
    for flag in ("license", "modelfile", "parameters", "template", "system"):
        p.add_argument(f"--{flag}", action="store_true")
    p.add_argument("-v", "--verbose", action="store_true")
    p.set_defaults(fn=cmd_show)
    p = sub.add_parser("run", help="Run a model")
    p.add_argument("model")
    p.add_argument("prompt", nargs="*")
    p.add_argument("--format", default="")
    p.add_argument("--keepalive", default="")
    p.add_argument("--think", default=None)
    p.add_argument("--insecure", action="store_true")
    p.add_argument("--verbose", action="store_true")
    p.set_defaults(fn=cmd_run)
    p = sub.add_parser("stop", help="Stop a running model")
    p.add_argument("model")
    p.set_defaults(fn=cmd_stop)
    for name, fn, hlp in (("pull", cmd_pull, "Pull a model from a registry"), ("push", cmd_push, "Push a model to a registry")):
        p = sub.add_parser(name, help=hlp)
        p.add_argument("model")
        p.add_argument("--insecure", action="store_true")
        p.set_defaults(fn=fn)
    sub.add_parser("list", aliases=["ls"], help="List models").set_defaults(fn=cmd_list)
    sub.add_parser("ps", help="List running models").set_defaults(fn=cmd_ps)
    p = sub.add_parser("cp", help="Copy a model")
    p.add_argument("source")
    p.add_argument("destination")
    p.set_defaults(fn=cmd_cp)
    p = sub.add_parser("rm", help="Remove a model")
    p.add_argument("models", nargs="+")
    p.set_defaults(fn=cmd_rm)
    p = sub.add_parser("bench", help="Benchmark models through the API")
    p.add_argument("--model", required=True, help="comma-separated model names")
    p.add_argument("--epochs", type=int, default=6)
    p.add_argument("--warmup", type=int, default=1)
    p.add_argument("--max-tokens", type=int, default=200)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--prompt", default="")
    p.add_argument("--prompt-tokens", type=int, default=64)
    p.add_argument("--keep-alive", default=None)
    p.add_argument("--format", default="benchstat", choices=["benchstat", "csv", "json"])
    p.set_defaults(fn=cmd_bench)
    sub.add_parser("gpu-discover", help="Print the devices this process can see as JSON").set_defaults(fn=cmd_gpu_discover)
    p = sub.add_parser("agent", help="Let a model work through tools (shell, files, skills) in this directory")
    p.add_argument("model")
    p.add_argument("prompt", nargs="*", help="one task; without it an interactive session starts")
    p.add_argument("--yes", action="store_true", help="allow every tool call without asking")
    p.add_argument("--skill", default="", help="load this skill before the first request")
    p.set_defaults(fn=cmd_agent)
    p = sub.add_parser("launch", help="Launch a coding tool connected to this server")
    p.add_argument("integration", nargs="?", help="claude, opencode, codex, droid (omit to pick from a list)")
    p.add_argument("--model", default=None, help="model to use (omit to reuse the last choice or pick from a list)")
    p.add_argument("--config", action="store_true", help="choose and save the model without starting the tool")
    p.add_argument("--dry-run", action="store_true", help="print the command line and environment instead of running them")
    p.set_defaults(fn=cmd_launch, extra=[])          # arguments after "--" go to the tool (split off in main)
    return ap


def cmd_agent(args) -> int:
    """A model working through tools in this directory: every change (shell command, file write) is asked about first
    unless ``--yes`` was given; "a" at the prompt allows that tool or exact command for the rest of the session."""
    from ..agent import Approval, Session, default_registry
    from ..agent.skills import SkillCatalog
    c = Client()
    info = c.show(args.model)
    if "tools" not in (info.get("capabilities") or []):
        print(f"Error: {args.model} does not support tools", file=sys.stderr)
        return 1
    ctx = next((int(v) for k, v in (info.get("model_info") or {}).items() if k.endswith(".context_length")), 0)

    def chat(**req):
        return c.request("POST", "/api/chat", req)

    def approver(calls, cwd):
        if args.yes:
            return Approval(True, allow_all=True)
        for k in calls:
            print(f"\n{k['name']} wants to run in {cwd}:\n  {json.dumps(k['args'], ensure_ascii=False)[:500]}", file=sys.stderr)
        print("Allow? [y]es / [a]lways for this / [n]o: ", end="", file=sys.stderr, flush=True)
        ans = sys.stdin.readline().strip().lower()
        if ans in ("a", "always"):
            return Approval(True, allow_scopes=[k["scope"] for k in calls])
        return Approval(ans in ("y", "yes"), reason="" if ans in ("y", "yes") else "declined at the prompt")

    def events(kind, data):
        if kind == "tool_start":
            print(f"\x1b[90m> {data['name']} {json.dumps(data['args'], ensure_ascii=False)[:200]}\x1b[0m", file=sys.stderr)
        elif kind in ("compacted", "denied"):
            print(f"\x1b[90m[{kind}]\x1b[0m", file=sys.stderr)

    skills = SkillCatalog()
    s = Session(chat, default_registry(skills), approver=approver, events=events, context_window=ctx, skills=skills)
    system = ("You are a coding assistant working in the user's directory through tools. Inspect before you change, make the smallest change "
              "that does the job, and say what you did." + ("\nSkills you can load with the skill tool:\n" + skills.describe() if skills.names() else ""))
    messages: list[dict[str, Any]] = []
    prompts = [" ".join(args.prompt)] if args.prompt else None
    while True:
        if prompts is not None:
            if not prompts:
                return 0
            text = prompts.pop(0)
        else:
            try:
                text = input(">>> ").strip()
            except (EOFError, KeyboardInterrupt):
                print()
                return 0
            if text in ("/bye", "/exit"):
                return 0
            if not text:
                continue
        r = s.run(args.model, messages + [{"role": "user", "content": text}], system=system, skill=args.skill or "")
        messages = [m for m in r.messages if m.get("role") != "system"]
        print(r.messages[-1].get("content", "") if r.stopped == "done" else f"[stopped: {r.stopped}]")


def cmd_launch(args) -> int:
    from .launch import launch
    extra = list(args.extra or [])
    return launch(Client(), args.integration, args.model, extra, choose_only=args.config, dry_run=args.dry_run)


def interactive_menu() -> int:
    """No command on a terminal: pick what to do (cmd/tui: the reference opens its launcher the same way)."""
    from . import tui
    from .launch import INTEGRATIONS, launch
    items = [tui.Item("run", "Chat with a model")] + [tui.Item(i.name, i.description) for i in INTEGRATIONS if not i.hidden]
    try:
        what = tui.select("What would you like to do?", items)
        if what != "run":
            return launch(Client(), what, None, [])
        models = [tui.Item(m["name"]) for m in Client().list().get("models", [])]
        if not models:
            print("No models are installed; pull one first (ollama pull <model>).", file=sys.stderr)
            return 1
        return main(["run", tui.select("Select a model:", models)])
    except tui.Cancelled:
        return 130


def main(argv: list[str] | None = None) -> int:
    ap = build_parser()
    argv = list(sys.argv[1:] if argv is None else argv)
    passthrough: list[str] = []
    if "launch" in argv[:1] and "--" in argv:
        cut = argv.index("--")
        argv, passthrough = argv[:cut], argv[cut + 1:]
    args = ap.parse_args(argv)
    if passthrough:
        args.extra = passthrough
    if args.version and not args.cmd:
        try:
            print(f"ollama-b200 version is {Client(timeout=2).version()}")
        except (ConnectionError, ResponseError):
            print(f"Warning: could not connect to a running server\nclient version is {VERSION}")
        return 0
    if not args.cmd:
        if sys.stdin.isatty() and sys.stdout.isatty():
            try:
                return interactive_menu()
            except (ConnectionError, ResponseError) as e:
                print(f"Error: {e}", file=sys.stderr)
                return 1
        ap.print_help()
        return 0
    try:
        return args.fn(args) or 0
    except ResponseError as e:
        print(f"Error: {e.message}", file=sys.stderr)
        return 1
    except ConnectionError as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    except KeyboardInterrupt:
        return 130


if __name__ == "__main__":
    sys.exit(main())
