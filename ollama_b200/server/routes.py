"""REST API: the public surface of the runtime (ASGI application).

Route table, status codes and streaming format follow the reference server (server/routes.go:1876-1926
routes; :2097-2144 NDJSON streaming; :3107-3120 error -> status mapping; :1776-1874 host allow-list and
CORS).  ``/api/tokenize`` and ``/api/detokenize`` are additions over that table; they expose the
runner's tokenizer calls (llm/server.go:68-69).
"""
from __future__ import annotations

import asyncio
import base64
import datetime
import hashlib
import json
import logging
import math
import os
import time
from typing import Any, AsyncIterator, Callable, Iterator

from starlette.applications import Starlette
from starlette.middleware import Middleware
from starlette.middleware.cors import CORSMiddleware
from starlette.requests import Request
from starlette.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse
from starlette.routing import Route

from .. import envconfig, version
from ..api.types import OptionError, default_options, options_from_map, parse_keep_alive, parse_think, think_enabled
from ..engine.grammar import GrammarError, grammar_for_format
from ..engine.runner import CompletionRequest, RunnerError
from ..engine.sampler import SamplingParams
from ..store import manifest as M
from ..store.create import CreateError, create_model
from ..store.model import CAP_COMPLETION, CAP_EMBEDDING, CAP_INSERT, CAP_THINKING, CAP_TOOLS, CAP_VISION, CapabilityError, Model, ModelNotFound, get_model
from ..store.names import parse_name
from ..text import harmony
from ..text.builtin import parser_for
from ..text.gotemplate import TemplateError
from ..text.thinking import ThinkingParser, infer_tags
from ..text.tools import ToolParser, infer_tag, tool_call_id
from .caches import InferenceModelCache, ModelListCache, ModelShowCache, RecommendationsCache
from .prompt import PromptRenderer, chat_prompt
from .sched import Scheduler, SchedulerError

log = logging.getLogger("ollama_b200.server")


class APIError(Exception):
    def __init__(self, status: int, msg: str):
        super().__init__(msg)
        self.status, self.msg = status, msg


def _now() -> str:
    return datetime.datetime.now(datetime.timezone.utc).astimezone().isoformat()


def _ns(seconds: float) -> int:
    return int(seconds * 1e9)


def _err(status: int, msg: str) -> JSONResponse:
    return JSONResponse({"error": msg}, status_code=status)


class Server:
    """Holds the scheduler and implements the handlers; ``app`` is the ASGI application."""

    def __init__(self, sched: Scheduler | None = None):
        from ..discover.devices import gpu_devices
        self.sched = sched or Scheduler(get_gpus_fn=gpu_devices)
        self.renderers: dict[str, PromptRenderer] = {}
        self.list_cache, self.show_cache = ModelListCache(), ModelShowCache()
        self.model_cache, self.recommendations = InferenceModelCache(), RecommendationsCache()
        from .request_log import RequestLogger
        self.request_log = RequestLogger()
        self.app = self._build()
        self.app.state.server = self        # tests and embedding programs reach the scheduler and the caches through the app

    # -- plumbing ---------------------------------------------------------------------------------------
    def _build(self) -> Starlette:
        r = [
            Route("/", self.root, methods=["GET", "HEAD"]),
            Route("/api/version", self.version, methods=["GET", "HEAD"]),
            Route("/api/status", self.status, methods=["GET"]),
            Route("/api/generate", self.generate, methods=["POST"]),
            Route("/api/chat", self.chat, methods=["POST"]),
            Route("/api/embed", self.embed, methods=["POST"]),
            Route("/api/embeddings", self.embeddings, methods=["POST"]),
            Route("/api/tokenize", self.tokenize, methods=["POST"]),
            Route("/api/detokenize", self.detokenize, methods=["POST"]),
            Route("/api/ps", self.ps, methods=["GET"]),
            Route("/metrics", self.metrics, methods=["GET"]),
            Route("/api/tags", self.tags, methods=["GET", "HEAD"]),
            Route("/api/show", self.show, methods=["POST"]),
            Route("/api/create", self.create, methods=["POST"]),
            Route("/api/copy", self.copy, methods=["POST"]),
            Route("/api/delete", self.delete, methods=["DELETE"]),
            Route("/api/pull", self.pull, methods=["POST"]),
            Route("/api/push", self.push, methods=["POST"]),
            Route("/api/blobs/{digest}", self.blob_head, methods=["HEAD"]),
            Route("/api/blobs/{digest}", self.blob_create, methods=["POST"]),
            Route("/api/me", self.cloud_stub, methods=["POST"]),
            Route("/api/signout", self.cloud_stub, methods=["POST"]),
            Route("/api/experimental/web_search", self.cloud_stub, methods=["POST"]),
            Route("/api/experimental/web_fetch", self.cloud_stub, methods=["POST"]),
            Route("/api/experimental/model-recommendations", self.model_recommendations, methods=["GET"]),
            Route("/api/user/keys/{key:path}", self.cloud_stub, methods=["DELETE"]),
        ]
        from .openai import openai_routes
        from .anthropic import anthropic_routes
        r += openai_routes(self) + anthropic_routes(self)
        origins = envconfig.allowed_origins()
        rx = "|".join(_origin_regex(o) for o in origins)
        mw = [Middleware(CORSMiddleware, allow_origin_regex=rx, allow_methods=["*"], allow_credentials=False,
                         allow_headers=["Authorization", "Content-Type", "User-Agent", "Accept", "X-Requested-With", "OpenAI-Beta",
                                        "x-stainless-arch", "x-stainless-async", "x-stainless-custom-poll-interval", "x-stainless-helper-method",
                                        "x-stainless-lang", "x-stainless-os", "x-stainless-package-version", "x-stainless-poll-helper",
                                        "x-stainless-retry-count", "x-stainless-runtime", "x-stainless-runtime-version", "x-stainless-timeout"]),
              Middleware(AllowedHosts)]
        app = Starlette(routes=r, middleware=mw, on_shutdown=[self.sched.unload_all])
        app.add_exception_handler(APIError, lambda req, e: _err(e.status, e.msg))
        return app

    async def model_recommendations(self, request: Request):
        """Cached list, refreshed behind the reader's back (server/routes.go:1931-1947)."""
        return JSONResponse({"recommendations": self.recommendations.get_swr()})

    async def _json(self, request: Request) -> dict[str, Any]:
        body = await request.body()
        if not body:
            raise APIError(400, "missing request body")
        self.request_log.record(request.url.path, body)
        try:
            d = json.loads(body)
        except ValueError as e:
            raise APIError(400, f"invalid JSON: {e}") from None
        if not isinstance(d, dict):
            raise APIError(400, "request body must be a JSON object")
        _check_types(d)
        return d

    def _model(self, name: str) -> Model:
        if not name:
            raise APIError(400, "model is required")
        try:
            return self.model_cache.get(name)
        except ModelNotFound:
            raise APIError(404, f"model '{name}' not found") from None

    def _options(self, model: Model, req_opts: dict[str, Any] | None) -> dict[str, Any]:
        opts = default_options()
        try:
            options_from_map(opts, model.options)
            options_from_map(opts, req_opts)
        except OptionError as e:
            raise APIError(400, str(e)) from None
        return opts

    def _schedule(self, model: Model, caps: tuple[str, ...], req_opts: dict[str, Any] | None, keep_alive: Any):
        try:
            model.check_capabilities(*caps)
        except CapabilityError as e:
            raise APIError(400, str(e)) from None
        opts = self._options(model, req_opts)
        try:
            ka = parse_keep_alive(keep_alive)
        except ValueError as e:
            raise APIError(400, str(e)) from None
        try:
            batch_auto = "num_batch" not in (model.options or {}) and "num_batch" not in (req_opts or {})
            ref = self.sched.get_runner(model, opts, ka, batch_auto=batch_auto)
        except SchedulerError as e:
            raise APIError(e.status, str(e)) from None
        return ref, opts

    @staticmethod
    def _refuse_images(model: Model, has_images: bool, runner: Any = None):
        """Image input: a model without a vision tower cannot take it (server/routes.go: images add the vision capability to the
        request); a vision checkpoint whose tower this engine does not run (anything but gemma3's, or a back end that takes no
        embeddings) is refused as well, never answered as if the images were not there.  Called before scheduling with the
        model only, and again with the loaded runner."""
        if not has_images:
            return None
        try:
            model.check_capabilities(CAP_VISION)
        except CapabilityError as e:
            return _err(400, str(e))
        if runner is not None and (not hasattr(runner, "vision") or runner.vision() is None):
            return _err(400, f"{model.short_name or model.name}: image input is not available: this engine runs the text path of this model only")
        return None

    @staticmethod
    def _image_bytes(images: list) -> list[bytes]:
        """API images (base64 text, or bytes from an in-process caller) -> encoded image bytes."""
        import base64
        out = []
        for im in images:
            out.append(bytes(im) if isinstance(im, (bytes, bytearray)) else base64.b64decode(str(im), validate=False))
        return out

    def _renderer(self, model: Model, runner: Any) -> PromptRenderer:
        key = model.digest or model.name
        r = self.renderers.get(key)
        if r is None:
            r = self.renderers[key] = PromptRenderer(model, getattr(runner, "tokenizer", None))
        return r

    @staticmethod
    def _sampling(opts: dict[str, Any], logprobs: bool = False, top_logprobs: int = 0) -> SamplingParams:
        return SamplingParams(temperature=opts["temperature"], top_k=opts["top_k"], top_p=opts["top_p"], min_p=opts["min_p"],
                              typical_p=opts["typical_p"], repeat_last_n=opts["repeat_last_n"], repeat_penalty=opts["repeat_penalty"],
                              presence_penalty=opts["presence_penalty"], frequency_penalty=opts["frequency_penalty"], seed=opts["seed"],
                              logprobs=logprobs, top_logprobs=top_logprobs)

    def _stream(self, gen: Callable[[], Iterator[dict[str, Any]]], stream: bool, ref=None, collapse: Callable | None = None):
        """NDJSON streaming, or one JSON object when ``stream`` is false; errors after the first chunk become a trailing line."""
        sched = self.sched

        def guarded() -> Iterator[dict[str, Any]]:
            try:
                yield from gen()
            except RunnerError as e:
                sched.expire_for_runtime_oom(e)       # a device that ran out of memory is emptied before the next request
                raise
            finally:
                if ref is not None:
                    sched.release(ref)

        if not stream:
            try:
                items = list(guarded())
            except RunnerError as e:
                return _err(e.status, str(e))
            except APIError as e:
                return _err(e.status, e.msg)
            out = collapse(items) if collapse else (items[-1] if items else {})
            return JSONResponse(out)

        def lines() -> Iterator[bytes]:
            try:
                for obj in guarded():
                    yield (json.dumps(obj, ensure_ascii=False) + "\n").encode()
            except (RunnerError, APIError, SchedulerError) as e:
                yield (json.dumps({"error": str(e)}) + "\n").encode()
            except Exception as e:  # keep the stream well-formed whatever happens
                log.exception("stream failed")
                yield (json.dumps({"error": str(e)}) + "\n").encode()

        return StreamingResponse(lines(), media_type="application/x-ndjson")

    # -- trivial routes ------------------------------------------------------------------------------------
    async def root(self, request: Request):
        return PlainTextResponse("Ollama is running")

    async def version(self, request: Request):
        return JSONResponse({"version": version.VERSION})

    async def status(self, request: Request):
        return JSONResponse({"cloud": {"disabled": True, "source": "local"}})

    async def cloud_stub(self, request: Request):
        return _err(501, "cloud features are not available in this runtime")

    # -- generate ------------------------------------------------------------------------------------------
    async def generate(self, request: Request):
        req = await self._json(request)
        return await asyncio.to_thread(self._generate, req)

    def _generate(self, req: dict[str, Any]):
        t_start = time.time()
        top_lp = int(req.get("top_logprobs") or 0)
        if top_lp < 0 or top_lp > 20:
            return _err(400, "top_logprobs must be between 0 and 20")
        name = req.get("model", "")
        model = self._model(name)
        prompt = req.get("prompt", "") or ""
        stream = req.get("stream", True) is not False
        try:
            ka = parse_keep_alive(req.get("keep_alive"))
            think = parse_think(req.get("think"))
        except ValueError as e:
            return _err(400, str(e))
        if prompt == "" and not req.get("context") and ka is not None and ka == 0 and not req.get("images"):
            self.sched.expire_runner(model)
            return JSONResponse({"model": name, "created_at": _now(), "response": "", "done": True, "done_reason": "unload"})
        caps = [CAP_COMPLETION]
        if req.get("suffix"):
            caps.append(CAP_INSERT)
        if think is not None and think_enabled(think):
            caps.append(CAP_THINKING)
        if req.get("raw") and (req.get("template") or req.get("system") or req.get("context")):
            return _err(400, "raw mode does not support template, system, or context")
        refusal = self._refuse_images(model, bool(req.get("images")))
        if refusal is not None:
            return refusal
        ref, opts = self._schedule(model, tuple(caps), req.get("options"), req.get("keep_alive"))
        runner = ref.runner
        t_loaded = time.time()
        media: list[bytes] = []
        if req.get("images"):
            refusal = self._refuse_images(model, True, runner)
            if refusal is not None:
                self.sched.release(ref)
                return refusal
            try:
                media = self._image_bytes(req["images"])
            except Exception:
                self.sched.release(ref)
                return _err(400, "invalid image data")
            if not req.get("raw") or "[img-" not in prompt:      # server/routes.go: every image gets its [img-N] marker in front of the prompt
                prompt = "".join(f"[img-{i}]" for i in range(len(media))) + prompt
        if prompt == "" and not req.get("context"):
            self.sched.release(ref)
            return JSONResponse({"model": name, "created_at": _now(), "response": "", "done": True, "done_reason": "load"})
        try:
            grammar = grammar_for_format(req.get("format"))
        except GrammarError as e:
            self.sched.release(ref)
            return _err(400, str(e))
        rend = self._renderer(model, runner)
        try:
            if req.get("raw"):
                text = prompt
            else:
                system = req.get("system") if req.get("system") is not None else model.system
                if model.messages and not req.get("context"):
                    msgs = list(model.messages) + ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": prompt}]
                    text = rend.render_chat(msgs, None, think)
                else:
                    text = rend.render_generate(system or "", prompt, req.get("suffix", "") or "", req.get("template"), think)
        except TemplateError as e:
            self.sched.release(ref)
            return _err(400, f"template error: {e}")
        if req.get("_debug_render_only"):
            self.sched.release(ref)
            return JSONResponse({"model": name, "created_at": _now(), "_debug_info": {"rendered_template": text}})
        tokens: Any = text
        if req.get("context"):
            tokens = [int(t) for t in req["context"]] + runner.tokenize(text, add_special=False)
        creq = CompletionRequest(prompt=tokens, sampling=self._sampling(opts, bool(req.get("logprobs")), top_lp), num_predict=opts["num_predict"],
                                 num_keep=opts["num_keep"], stop=list(opts.get("stop") or []), grammar=grammar,
                                 grammar_after="" if req.get("raw") else self._grammar_gate(rend, grammar, think, text),
                                 truncate=req.get("truncate", True) is not False, shift=req.get("shift", True) is not False,
                                 preserved_tokens=rend.is_harmony, images=media if isinstance(tokens, str) else [])
        tp = self._thinking_parser(rend, think, text) if not req.get("raw") else None
        # a model may name the harmony parser although it brings a template of its own (model/parsers/parsers.go:69-70)
        use_harmony = rend.is_harmony or model.config.get("parser") == "harmony"
        hp = harmony.HarmonyParser(rend.names) if use_harmony and not req.get("raw") else None
        bp = parser_for(model.config.get("parser"), None, think) if hp is None and not req.get("raw") else None

        def gen() -> Iterator[dict[str, Any]]:
            out_tokens: list[int] = []
            for ch in runner.completion(creq):
                out_tokens += ch.tokens
                content, thinking = ch.content, ""
                if hp is not None:
                    thinking, content, _ = hp.add(content)
                elif bp is not None:        # the model names a built-in parser (Modelfile PARSER)
                    try:
                        content, thinking, _ = bp.add(content, ch.done)
                    except ValueError as e:     # a call block the parser cannot read fails the request (server/routes.go:686-690, :2810-2814)
                        raise APIError(500, str(e)) from e
                elif tp is not None:
                    thinking, content = tp.add(content)
                if think is not None and not think_enabled(think):
                    thinking = ""
                if ch.done:
                    final = {"model": name, "created_at": _now(), "response": content, "done": True, "done_reason": ch.done_reason,
                             "total_duration": _ns(time.time() - t_start), "load_duration": _ns(t_loaded - t_start),
                             "prompt_eval_count": ch.prompt_eval_count, "prompt_eval_duration": _ns(ch.prompt_eval_duration),
                             "eval_count": ch.eval_count, "eval_duration": _ns(ch.eval_duration)}
                    if thinking:
                        final["thinking"] = thinking
                    if not req.get("raw"):
                        base = tokens if isinstance(tokens, list) else runner.tokenize(text, add_special=True)
                        final["context"] = list(base) + out_tokens
                    yield final
                elif content or thinking or ch.logprobs:
                    obj = {"model": name, "created_at": _now(), "response": content, "done": False}
                    if thinking:
                        obj["thinking"] = thinking
                    if ch.logprobs:
                        obj["logprobs"] = _logprobs_json(runner, ch.logprobs)
                    yield obj

        def collapse(items: list[dict[str, Any]]) -> dict[str, Any]:
            final = dict(items[-1]) if items else {}
            final["response"] = "".join(i.get("response", "") for i in items)
            th = "".join(i.get("thinking", "") for i in items)
            if th:
                final["thinking"] = th
            lps = [lp for i in items for lp in i.get("logprobs", [])]
            if lps:
                final["logprobs"] = lps
            return final

        return self._stream(gen, stream, ref, collapse)

    def _grammar_gate(self, rend: PromptRenderer, grammar: str | None, think: Any, prompt_text: str) -> str:
        """Text after which a structured-output grammar starts to apply: the end of the reasoning block when the model
        reasons first (a prompt that ends inside the block, or harmony's analysis channel), "" otherwise."""
        if not grammar or not (think is None or think_enabled(think)):
            return ""
        if rend.is_harmony:
            return "<|channel|>final<|message|>"
        tp = self._thinking_parser(rend, think, prompt_text)
        if tp is not None and prompt_text.rstrip().endswith(tp.opening):
            return tp.closing
        return ""

    def _thinking_parser(self, rend: PromptRenderer, think: Any, prompt_text: str) -> ThinkingParser | None:
        if rend.is_harmony:
            return None
        src = rend.template_source
        o, c = infer_tags(src) if rend.go_template is not None else ("", "")
        if not o and ("<think>" in src or "enable_thinking" in src or "reasoning_content" in src):
            o, c = "<think>", "</think>"
        if not o:
            return None
        if think is not None and not think_enabled(think) and rend.go_template is None:
            return None
        return ThinkingParser(o, c, started=prompt_text.rstrip().endswith(o))

    # -- chat ----------------------------------------------------------------------------------------------
    async def chat(self, request: Request):
        req = await self._json(request)
        return await asyncio.to_thread(self._chat, req)

    def _chat(self, req: dict[str, Any]):
        t_start = time.time()
        top_lp = int(req.get("top_logprobs") or 0)
        if top_lp < 0 or top_lp > 20:
            return _err(400, "top_logprobs must be between 0 and 20")
        name = req.get("model", "")
        model = self._model(name)
        stream = req.get("stream", True) is not False
        messages = req.get("messages") or []
        if not isinstance(messages, list):
            return _err(400, "messages must be an array")
        tools = req.get("tools") or []
        try:
            ka = parse_keep_alive(req.get("keep_alive"))
            think = parse_think(req.get("think"))
        except ValueError as e:
            return _err(400, str(e))
        if not messages and ka is not None and ka == 0:
            self.sched.expire_runner(model)
            return JSONResponse({"model": name, "created_at": _now(), "message": {"role": "assistant", "content": ""}, "done": True,
                                 "done_reason": "unload"})
        caps = [CAP_COMPLETION]
        if tools:
            caps.append(CAP_TOOLS)
        if think is not None and think_enabled(think):
            caps.append(CAP_THINKING)
        refusal = self._refuse_images(model, any(m.get("images") for m in messages if isinstance(m, dict)))
        if refusal is not None:
            return refusal
        ref, opts = self._schedule(model, tuple(caps), req.get("options"), req.get("keep_alive"))
        runner = ref.runner
        t_loaded = time.time()
        if not messages:
            self.sched.release(ref)
            return JSONResponse({"model": name, "created_at": _now(), "message": {"role": "assistant", "content": ""}, "done": True,
                                 "done_reason": "load"})
        try:
            grammar = grammar_for_format(req.get("format"))
        except GrammarError as e:
            self.sched.release(ref)
            return _err(400, str(e))
        rend = self._renderer(model, runner)
        msgs = list(model.messages) + [{**m, "role": str(m.get("role", "")).lower()} for m in messages]     # roles compare in lower case
        media: list[bytes] = []
        if any(m.get("images") for m in msgs):
            refusal = self._refuse_images(model, True, runner)
            if refusal is not None:
                self.sched.release(ref)
                return refusal
            from ..text.renderers import image_tagged
            try:
                for i, m in enumerate(msgs):        # every image gets its [img-N] marker in the message it came with (server/prompt.go:96-133)
                    imgs = m.get("images") or []
                    if imgs:
                        msgs[i] = {**m, "content": image_tagged(m.get("content", "") or "", len(imgs), len(media))}
                        media += self._image_bytes(imgs)
            except Exception:
                self.sched.release(ref)
                return _err(400, "invalid image data")
        if model.system and not any(m.get("role") == "system" for m in msgs):
            msgs.insert(0, {"role": "system", "content": model.system})
        if think == "max" and rend.is_harmony:
            think = "high"
        # earlier assistant turns of reasoning models are stored without their reasoning block
        if rend.go_template is None and not rend.is_harmony:
            for m in msgs[:-1]:
                if m.get("role") == "assistant" and "</think>" in m.get("content", ""):
                    m["content"] = m["content"].split("</think>", 1)[1].lstrip()
        try:
            # an image counts as 768 tokens when the conversation is cut to fit (server/prompt.go:29-33)
            text, _ = chat_prompt(lambda ms: rend.render_chat(ms, tools, think),
                                  lambda s: len(runner.tokenize(s, add_special=True)) + 768 * s.count("[img-"),
                                  msgs, runner.n_ctx, req.get("truncate", True) is not False)
        except TemplateError as e:
            self.sched.release(ref)
            return _err(400, f"template error: {e}")
        if req.get("_debug_render_only"):
            self.sched.release(ref)
            return JSONResponse({"model": name, "created_at": _now(), "_debug_info": {"rendered_template": text}})
        # structured output of a reasoning model: the reasoning stays free-form, the grammar applies to the answer
        # (the reference re-issues the request once the reasoning ended, server/routes.go:2910-2935; here the runner arms
        # the grammar when the end of the reasoning block shows up in the output)
        gate = self._grammar_gate(rend, grammar, think, text)
        creq = CompletionRequest(prompt=text, sampling=self._sampling(opts, bool(req.get("logprobs")), top_lp), num_predict=opts["num_predict"],
                                 num_keep=opts["num_keep"], stop=list(opts.get("stop") or []), grammar=grammar, grammar_after=gate,
                                 truncate=req.get("truncate", True) is not False, shift=req.get("shift", True) is not False,
                                 preserved_tokens=rend.is_harmony, images=media)
        hp = harmony.HarmonyParser(rend.names) if rend.is_harmony or model.config.get("parser") == "harmony" else None
        prefill = msgs[-1].get("content", "") if msgs and msgs[-1].get("role") == "assistant" else ""
        after_tool = bool(msgs) and msgs[-1].get("role") == "tool"
        bp = parser_for(model.config.get("parser"), tools, think, prefill, after_tool) if hp is None else None
        tp = self._thinking_parser(rend, think, text) if bp is None else None
        tool_parser = ToolParser(tools, infer_tag(rend.template_source)) if tools and hp is None and bp is None else None
        show_thinking = think is None or think_enabled(think)

        n_calls = 0

        def gen() -> Iterator[dict[str, Any]]:
            nonlocal n_calls
            for ch in runner.completion(creq):
                content, thinking, calls = ch.content, "", []
                if hp is not None:
                    thinking, content, calls = hp.add(content)
                elif bp is not None:
                    try:
                        content, thinking, calls = bp.add(content, ch.done)
                    except ValueError as e:     # a call block the parser cannot read fails the request (server/routes.go:686-690, :2810-2814)
                        raise APIError(500, str(e)) from e
                    for c in calls:         # calls of the built-in parsers get their id and running index here
                        c.setdefault("id", tool_call_id())
                        c["function"].setdefault("index", n_calls)
                        n_calls += 1
                else:
                    if tp is not None:
                        thinking, content = tp.add(content)
                    if tool_parser is not None and content:
                        calls, content = tool_parser.add(content)
                if not show_thinking:
                    thinking = ""
                msg: dict[str, Any] = {"role": "assistant", "content": content}
                if thinking:
                    msg["thinking"] = thinking
                if calls:
                    msg["tool_calls"] = calls
                if ch.done:
                    if tool_parser is not None:
                        msg["content"] += tool_parser.flush()
                    final = {"model": name, "created_at": _now(), "message": msg, "done": True, "done_reason": ch.done_reason,
                             "total_duration": _ns(time.time() - t_start), "load_duration": _ns(t_loaded - t_start),
                             "prompt_eval_count": ch.prompt_eval_count, "prompt_eval_duration": _ns(ch.prompt_eval_duration),
                             "eval_count": ch.eval_count, "eval_duration": _ns(ch.eval_duration)}
                    yield final
                elif content or thinking or calls or ch.logprobs:
                    obj = {"model": name, "created_at": _now(), "message": msg, "done": False}
                    if ch.logprobs:
                        obj["logprobs"] = _logprobs_json(runner, ch.logprobs)
                    yield obj

        def collapse(items: list[dict[str, Any]]) -> dict[str, Any]:
            final = dict(items[-1]) if items else {}
            msg = {"role": "assistant", "content": "".join(i["message"].get("content", "") for i in items)}
            th = "".join(i["message"].get("thinking", "") for i in items)
            if th:
                msg["thinking"] = th
            calls = [c for i in items for c in i["message"].get("tool_calls", [])]
            if calls:
                msg["tool_calls"] = calls
            final["message"] = msg
            lps = [lp for i in items for lp in i.get("logprobs", [])]
            if lps:
                final["logprobs"] = lps
            return final

        return self._stream(gen, stream, ref, collapse)

    # -- embeddings ----------------------------------------------------------------------------------------
    async def embed(self, request: Request):
        req = await self._json(request)
        return await asyncio.to_thread(self._embed, req, False)

    async def embeddings(self, request: Request):
        req = await self._json(request)
        return await asyncio.to_thread(self._embed, req, True)

    def _embed(self, req: dict[str, Any], legacy: bool):
        t_start = time.time()
        name = req.get("model", "")
        model = self._model(name)
        inp = req.get("prompt") if legacy else req.get("input")
        if inp is None or inp == "" or inp == []:
            if legacy:
                return JSONResponse({"embedding": []})
            return JSONResponse({"model": name, "embeddings": []})
        inputs = [inp] if isinstance(inp, str) else list(inp)
        if not all(isinstance(s, str) for s in inputs):
            return _err(400, "invalid input type")
        ref, opts = self._schedule(model, (), req.get("options"), req.get("keep_alive"))
        runner = ref.runner
        t_loaded = time.time()
        try:
            truncate = req.get("truncate", True) is not False
            vecs, count = [], 0
            for s in inputs:
                toks = runner.tokenize(s, add_special=True)
                limit = runner.n_ctx - 1
                if len(toks) > limit:
                    if not truncate:
                        return _err(400, "input exceeds maximum context length")
                    toks = toks[:limit]
                v, n = runner.embedding(toks)
                count += n
                vecs.append(_normalize(v, req.get("dimensions") or 0))
        except RunnerError as e:
            return _err(e.status, str(e))
        finally:
            self.sched.release(ref)
        if legacy:
            return JSONResponse({"embedding": vecs[0]})
        return JSONResponse({"model": name, "embeddings": vecs, "total_duration": _ns(time.time() - t_start),
                             "load_duration": _ns(t_loaded - t_start), "prompt_eval_count": count})

    # -- tokenize / detokenize -----------------------------------------------------------------------------
    async def tokenize(self, request: Request):
        req = await self._json(request)
        return await asyncio.to_thread(self._tok, req, True)

    async def detokenize(self, request: Request):
        req = await self._json(request)
        return await asyncio.to_thread(self._tok, req, False)

    def _tok(self, req: dict[str, Any], encode: bool):
        model = self._model(req.get("model", ""))
        ref, _ = self._schedule(model, (), req.get("options"), req.get("keep_alive"))
        try:
            if encode:
                text = req.get("content", req.get("text", ""))
                if not isinstance(text, str):
                    return _err(400, "content must be a string")
                return JSONResponse({"tokens": ref.runner.tokenize(text, add_special=bool(req.get("add_special", False)))})
            toks = req.get("tokens")
            if not isinstance(toks, list) or not all(isinstance(t, int) for t in toks):
                return _err(400, "tokens must be an array of integers")
            return JSONResponse({"content": ref.runner.detokenize(toks)})
        except RunnerError as e:
            return _err(e.status, str(e))
        finally:
            self.sched.release(ref)

    async def metrics(self, request: Request):
        """Prometheus text exposition of the loaded runners' totals (the reference exposes per-response durations and
        /api/ps only; this adds queue wait, time to first token and per-phase seconds per model for a scraper)."""
        lines: list[str] = []
        seen: set[str] = set()

        def emit(name: str, kind: str, help_: str, labels: dict[str, str], value: float) -> None:
            if name not in seen:
                seen.add(name)
                lines.append(f"# HELP {name} {help_}")
                lines.append(f"# TYPE {name} {kind}")
            lab = ",".join('%s="%s"' % (k, str(v).replace("\\", "\\\\").replace('"', '\\"')) for k, v in labels.items())
            lines.append(f"{name}{{{lab}}} {value:g}" if lab else f"{name} {value:g}")

        refs = self.sched.ps()
        emit("ollama_b200_loaded_models", "gauge", "Models currently loaded.", {}, len(refs))
        help_ = {"requests": "Completed requests.", "prompt_tokens": "Prompt tokens of completed requests.",
                 "cached_prompt_tokens": "Prompt tokens served from a slot's cached prefix.", "generated_tokens": "Generated tokens.",
                 "queue_seconds": "Seconds requests waited for a slot.", "prefill_seconds": "Seconds spent evaluating prompts.",
                 "decode_seconds": "Seconds spent generating (per sequence).", "ttft_seconds": "Sum of times from submission to first token.",
                 "decode_steps": "Decode steps run.", "decode_step_sequences": "Sequences advanced, summed over decode steps.",
                 "context_shifts": "Context shifts performed."}
        for r in refs:
            labels = {"model": getattr(r.model, "short_name", "") or getattr(r.model, "name", "")}
            emit("ollama_b200_model_vram_bytes", "gauge", "Device memory held by the model.", labels, float(r.vram_size))
            emit("ollama_b200_model_context_length", "gauge", "Context length per slot.", labels, float(r.context_length))
            stats = getattr(r.runner, "stats", None) or {}
            for k, v in stats.items():
                emit(f"ollama_b200_{k}_total", "counter", help_.get(k, k), labels, float(v))
            for reason, n in (getattr(r.runner, "done_reasons", None) or {}).items():
                emit("ollama_b200_done_total", "counter", "Completed requests by done_reason.", {**labels, "reason": reason}, float(n))
        return PlainTextResponse("\n".join(lines) + "\n", media_type="text/plain; version=0.0.4")

    # -- model management -----------------------------------------------------------------------------------
    async def ps(self, request: Request):
        models = []
        for r in self.sched.ps():
            m = r.model
            exp = "0001-01-01T00:00:00Z" if not math.isfinite(r.expires_at) else \
                (datetime.datetime.now(datetime.timezone.utc) + datetime.timedelta(seconds=max(0.0, r.expires_at - self.sched.now()))).isoformat()
            if not math.isfinite(r.expires_at):
                exp = (datetime.datetime.now(datetime.timezone.utc) + datetime.timedelta(days=365 * 100)).isoformat()
            models.append({"name": getattr(m, "short_name", ""), "model": getattr(m, "short_name", ""), "size": r.total_size,
                           "digest": getattr(m, "digest", ""), "details": _details(m), "expires_at": exp, "size_vram": r.vram_size,
                           "context_length": r.context_length})
        return JSONResponse({"models": models})

    async def tags(self, request: Request):
        def entry(n, man):
            cfg = man.config_json()
            return {"name": n.display(), "model": n.display(),
                    "modified_at": datetime.datetime.fromtimestamp(man.mtime, datetime.timezone.utc).isoformat(),
                    "size": man.size(), "digest": man.digest,
                    "details": {"parent_model": "", "format": cfg.get("model_format", ""), "family": cfg.get("model_family", ""),
                                "families": cfg.get("model_families"), "parameter_size": cfg.get("model_type", ""),
                                "quantization_level": cfg.get("file_type", "")}}

        def work():
            out = self.list_cache.list(entry)        # unchanged manifests are not read again
            out.sort(key=lambda m: m["modified_at"], reverse=True)
            return out
        return JSONResponse({"models": await asyncio.to_thread(work)})

    async def show(self, request: Request):
        req = await self._json(request)
        name = req.get("model") or req.get("name") or ""
        model = self._model(name)
        use_cache = ModelShowCache.cacheable(req)
        if use_cache:
            hit = self.show_cache.get(model.name, bool(req.get("verbose")), model.digest)
            if hit is not None:
                return JSONResponse(hit)

        def work():
            kv = dict(model.kv())
            tensors = kv.pop("__tensors__", [])
            info = {}
            for k, v in kv.items():
                if hasattr(v, "tolist"):
                    v = v.tolist()
                elif v.__class__.__name__ == "_ElidedArray":
                    v = None
                info[k] = v
            if req.get("system"):
                model.system = req["system"]
            params = []
            for k in sorted(model.options):
                v = model.options[k]
                for item in (v if isinstance(v, list) else [v]):
                    params.append(f"{k:<30} {json.dumps(item) if isinstance(item, str) else item}")
            out = {"license": "\n".join(model.license), "modelfile": model.modelfile(), "parameters": "\n".join(params),
                   "template": model.template or model.chat_template(), "system": model.system, "details": _details(model),
                   "messages": model.messages, "model_info": info, "capabilities": model.capabilities(),
                   "modified_at": datetime.datetime.fromtimestamp(model.mtime, datetime.timezone.utc).isoformat()}
            if model.config.get("renderer"):
                out["renderer"] = model.config["renderer"]
            if model.config.get("parser"):
                out["parser"] = model.config["parser"]
            if req.get("verbose"):
                out["tensors"] = [{"name": n, "type": t, "shape": s} for n, t, s in tensors]
            if use_cache:
                self.show_cache.put(model.name, bool(req.get("verbose")), model.digest, out)
            return out

        return JSONResponse(await asyncio.to_thread(work))

    async def create(self, request: Request):
        req = await self._json(request)
        stream = req.get("stream", True) is not False

        def gen():
            try:
                yield from create_model(req)
            except CreateError as e:
                raise APIError(e.status, str(e)) from None
            except M.StoreError as e:
                raise APIError(400, str(e)) from None

        if not stream:
            try:
                items = await asyncio.to_thread(lambda: list(gen()))
            except APIError as e:
                return _err(e.status, e.msg)
            return JSONResponse(items[-1])
        return self._stream(gen, True)

    async def copy(self, request: Request):
        req = await self._json(request)
        src, dst = parse_name(req.get("source") or ""), parse_name(req.get("destination") or "")
        if not src.valid:
            return _err(400, f"source {req.get('source')!r} is invalid")
        if not dst.valid:
            return _err(400, f"destination {req.get('destination')!r} is invalid")
        try:
            M.copy_model(src, dst)
        except M.StoreError:
            return _err(404, f"model {req.get('source')!r} not found")
        return Response(status_code=200)

    async def delete(self, request: Request):
        req = await self._json(request)
        name = parse_name(req.get("model") or req.get("name") or "")
        if not name.valid:
            return _err(400, "invalid model name")
        try:
            try:
                self.sched.expire_runner(get_model(str(name)))
            except ModelNotFound:
                pass
            M.delete_model(name)
        except M.StoreError:
            return _err(404, f"model '{req.get('model') or req.get('name')}' not found")
        return Response(status_code=200)

    async def pull(self, request: Request):
        req = await self._json(request)
        from ..store.registry import RegistryError, pull_model
        name = req.get("model") or req.get("name") or ""

        def gen():
            try:
                yield from pull_model(name, insecure=bool(req.get("insecure")))
            except RegistryError as e:
                raise APIError(e.status, str(e)) from None

        return self._stream(gen, req.get("stream", True) is not False)

    async def push(self, request: Request):
        req = await self._json(request)
        from ..store.registry import RegistryError, push_model
        name = req.get("model") or req.get("name") or ""

        def gen():
            try:
                yield from push_model(name, insecure=bool(req.get("insecure")))
            except RegistryError as e:
                raise APIError(e.status, str(e)) from None

        return self._stream(gen, req.get("stream", True) is not False)

    async def blob_head(self, request: Request):
        try:
            p = M.blob_path(request.path_params["digest"])
        except M.StoreError as e:
            return _err(400, str(e))
        return Response(status_code=200 if os.path.exists(p) else 404)

    async def blob_create(self, request: Request):
        digest = request.path_params["digest"]
        try:
            p = M.blob_path(digest)
        except M.StoreError as e:
            return _err(400, str(e))
        if os.path.exists(p):
            return Response(status_code=200)
        h = hashlib.sha256()
        tmp = p + f"-upload-{os.getpid()}-{time.time_ns()}"
        with open(tmp, "wb") as f:
            async for chunk in request.stream():
                f.write(chunk)
                h.update(chunk)
        if "sha256:" + h.hexdigest() != digest.replace("-", ":", 1):
            os.unlink(tmp)
            return _err(400, "digest does not match body")
        os.replace(tmp, p)
        return Response(status_code=201)


# ---------------------------------------------------------------------------------------------------------
def _is_num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and v == v and abs(v) != math.inf


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


# JSON kinds of the request fields of the native routes (api/types.go: a value of another kind fails to decode there)
_FIELD_KINDS: dict[str, tuple[str, Callable[[Any], bool]]] = {
    **{k: ("a string", lambda v: isinstance(v, str)) for k in (
        "model", "name", "prompt", "suffix", "system", "template", "from", "quantize", "quantization", "source", "destination", "content",
        "renderer", "parser", "draft_quantize")},
    **{k: ("a boolean", lambda v: isinstance(v, bool)) for k in (
        "stream", "raw", "verbose", "insecure", "truncate", "shift", "logprobs", "add_special")},
    **{k: ("an object", lambda v: isinstance(v, dict)) for k in ("options", "parameters", "files", "adapters", "draft_files", "drafts")},
    **{k: ("an array of objects", lambda v: isinstance(v, list) and all(isinstance(x, dict) for x in v)) for k in ("messages", "tools")},
    **{k: ("an array of integers", lambda v: isinstance(v, list) and all(_is_int(x) for x in v)) for k in ("context", "tokens")},
    "images": ("an array of strings", lambda v: isinstance(v, list) and all(isinstance(x, str) for x in v)),
    "format": ("a string or an object", lambda v: isinstance(v, (str, dict))),
    "keep_alive": ("a duration string or a number", lambda v: isinstance(v, str) or _is_num(v)),
    "think": ("a boolean or a string", lambda v: isinstance(v, (bool, str))),
    "top_logprobs": ("an integer", _is_int),
    "dimensions": ("an integer", _is_int),
    "input": ("a string or an array of strings", lambda v: isinstance(v, str) or (isinstance(v, list) and all(isinstance(x, str) for x in v))),
    "license": ("a string or an array of strings", lambda v: isinstance(v, str) or (isinstance(v, list) and all(isinstance(x, str) for x in v))),
}


def _check_types(req: dict[str, Any]) -> None:
    """400 for a field whose JSON kind is not the one the API defines (null counts as absent)."""
    for k, v in req.items():
        spec = _FIELD_KINDS.get(k)
        if spec is not None and v is not None and not spec[1](v):
            raise APIError(400, f"invalid request: {k!r} must be {spec[0]}")
    for m in req.get("messages") or []:
        for fk, ok, what in (("role", lambda v: isinstance(v, str), "a string"), ("content", lambda v: isinstance(v, str), "a string"),
                             ("thinking", lambda v: isinstance(v, str), "a string"),
                             ("tool_calls", lambda v: isinstance(v, list) and all(isinstance(x, dict) and isinstance(x.get("function"), dict) for x in v),
                              "an array of tool calls"),
                             ("images", lambda v: isinstance(v, list), "an array")):
            if m.get(fk) is not None and not ok(m[fk]):
                raise APIError(400, f"invalid request: message field {fk!r} must be {what}")
    for t in req.get("tools") or []:
        f = t.get("function")
        if not isinstance(f, dict) or not isinstance(f.get("name"), str) or not isinstance(f.get("parameters") or {}, dict):
            raise APIError(400, "invalid request: every tool needs a function object with a name")


def _details(m: Any) -> dict[str, Any]:
    cfg = getattr(m, "config", {}) or {}
    return {"parent_model": getattr(m, "parent_model", ""), "format": cfg.get("model_format", ""), "family": cfg.get("model_family", ""),
            "families": cfg.get("model_families"), "parameter_size": cfg.get("model_type", ""), "quantization_level": cfg.get("file_type", "")}


def _normalize(v: list[float], dims: int = 0) -> list[float]:
    if dims and 0 < dims < len(v):
        v = v[:dims]
    n = math.sqrt(sum(x * x for x in v))
    return [x / n for x in v] if n > 0 else list(v)


def _logprobs_json(runner: Any, lps) -> list[dict[str, Any]]:
    tk = runner.tokenizer

    def ent(tok: int, lp: float) -> dict[str, Any]:
        b = tk.token_bytes(tok) if tk is not None and 0 <= tok < tk.n_vocab else b""
        return {"token": b.decode("utf-8", errors="replace"), "logprob": lp, "bytes": list(b)}

    out = []
    for lp in lps:
        e = ent(lp.token, lp.logprob)
        if lp.top:
            e["top_logprobs"] = [ent(t, p) for t, p in lp.top]
        out.append(e)
    return out


def _origin_regex(origin: str) -> str:
    import re
    return "^" + re.escape(origin).replace(r"\*", ".*") + "$"


class AllowedHosts:
    """Reject requests whose Host header is not local when the server is bound to a loopback address
    (DNS-rebinding protection; server/routes.go:1776-1839)."""

    def __init__(self, app):
        self.app = app

    async def __call__(self, scope, receive, send):
        if scope["type"] != "http":
            return await self.app(scope, receive, send)
        bind = envconfig.host().host
        if bind not in ("127.0.0.1", "localhost", "::1"):
            return await self.app(scope, receive, send)
        host = ""
        for k, v in scope.get("headers", []):
            if k == b"host":
                host = v.decode("latin-1")
        h = host.rsplit(":", 1)[0].strip("[]") if host else ""
        ok = (h == "" or h in ("localhost", "127.0.0.1", "::1", "0.0.0.0", "testserver") or h.endswith((".localhost", ".local", ".internal"))
              or _is_ip(h) and (h.startswith("127.") or _is_private(h)) or h == os.uname().nodename)
        if not ok:
            resp = JSONResponse({"error": "forbidden"}, status_code=403)
            return await resp(scope, receive, send)
        return await self.app(scope, receive, send)


def _is_ip(h: str) -> bool:
    import ipaddress
    try:
        ipaddress.ip_address(h)
        return True
    except ValueError:
        return False


def _is_private(h: str) -> bool:
    import ipaddress
    try:
        a = ipaddress.ip_address(h)
        return a.is_private or a.is_loopback or a.is_unspecified
    except ValueError:
        return False


def create_app(sched: Scheduler | None = None) -> Starlette:
    return Server(sched).app
