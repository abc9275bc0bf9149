"""OpenAI-compatible routes, implemented as request / response rewriting around the native handlers.

``/v1/chat/completions``, ``/v1/completions``, ``/v1/embeddings``, ``/v1/models``, ``/v1/models/{model}``
and ``/v1/responses`` (the reference registers the same façade as middleware, server/routes.go:1916-1923;
conversions in openai/openai.go:269-507 and :549-864).  Streaming uses server-sent events with a final
``data: [DONE]``.
"""
from __future__ import annotations

import asyncio
import base64
import json
import struct
import time
import uuid
from typing import Any, AsyncIterator

from starlette.requests import Request
from starlette.responses import JSONResponse, StreamingResponse
from starlette.routing import Route

from ..store import manifest as M


def _oa_err(status: int, msg: str, typ: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"error": {"message": msg, "type": typ, "param": None, "code": None}}, status_code=status)


def _options(req: dict[str, Any]) -> dict[str, Any]:
    o: dict[str, Any] = {}
    if req.get("max_completion_tokens") is not None:
        o["num_predict"] = req["max_completion_tokens"]
    elif req.get("max_tokens") is not None:
        o["num_predict"] = req["max_tokens"]
    if req.get("temperature") is not None:
        o["temperature"] = req["temperature"]
    else:
        o["temperature"] = 1.0
    if req.get("top_p") is not None:
        o["top_p"] = req["top_p"]
    else:
        o["top_p"] = 1.0
    for k in ("seed", "frequency_penalty", "presence_penalty"):
        if req.get(k) is not None:
            o[k] = req[k]
    stop = req.get("stop")
    if isinstance(stop, str):
        o["stop"] = [stop]
    elif isinstance(stop, list):
        o["stop"] = stop
    return o


def _messages(req: dict[str, Any]) -> list[dict[str, Any]]:
    out = []
    call_names: dict[str, str] = {}        # id of an earlier call -> its function, to name a tool answer that only gives the id
    for m in req.get("messages") or []:
        role = m.get("role", "")
        if role == "developer":
            role = "system"
        content = m.get("content")
        images: list[str] = []
        if isinstance(content, list):
            texts = []
            for part in content:
                if part.get("type") == "text":
                    texts.append(part.get("text", ""))
                elif part.get("type") == "image_url":
                    url = (part.get("image_url") or {}).get("url", "")
                    if url.startswith("data:") and "," in url:
                        images.append(url.split(",", 1)[1])
                    else:
                        raise ValueError("invalid image input")
            content = "".join(texts)
        d: dict[str, Any] = {"role": role, "content": content or ""}
        if images:
            d["images"] = images
        if m.get("reasoning") or m.get("reasoning_content"):
            d["thinking"] = m.get("reasoning") or m.get("reasoning_content")
        if m.get("tool_calls"):
            calls = []
            for tc in m["tool_calls"]:
                fn = tc.get("function", {})
                args = fn.get("arguments")
                if isinstance(args, str):
                    try:
                        args = json.loads(args or "{}")
                    except ValueError:
                        raise ValueError("invalid tool call arguments") from None
                calls.append({"id": tc.get("id", ""), "function": {"name": fn.get("name", ""), "arguments": args or {}}})
                if tc.get("id"):
                    call_names[tc["id"]] = fn.get("name", "")
            d["tool_calls"] = calls
        if role == "tool":
            d["tool_call_id"] = m.get("tool_call_id", "")
            d["tool_name"] = m.get("name") or call_names.get(d["tool_call_id"], "")
        out.append(d)
    return out


def _finish(reason: str, has_tools: bool) -> str:
    """Finish reason of a whole answer: calls turn "stop" into "tool_calls"; any other reason (length, ...) passes through."""
    reason = reason or "stop"
    return "tool_calls" if reason == "stop" and has_tools else reason


class ChatStreamState:
    """What a chat stream remembers between native responses: whether the role went out and whether a call was sent."""

    def __init__(self):
        self.first_sent = False
        self.tool_sent = False


def chat_stream_frames(state: ChatStreamState, obj: dict[str, Any], base: dict[str, Any], want_usage: bool) -> list[dict[str, Any]]:
    """Chunks of an OpenAI chat stream for one native response (middleware/openai.go:80-164, openai/openai.go:344-395 of the
    reference).  The role is on the first chunk only; reasoning that arrives together with content or calls goes out as a chunk
    of its own first; the closing response with an empty message adds no empty content chunk; the finish reason has its own
    chunk with an empty delta ("tool_calls" replaces "stop" once a call was streamed, other reasons pass through); the usage
    chunk, when asked for, has an empty choices list."""
    msg = obj.get("message") or {}
    content, thinking, calls = msg.get("content", "") or "", msg.get("thinking", "") or "", msg.get("tool_calls") or []
    done = bool(obj.get("done"))
    frames: list[dict[str, Any]] = []
    trailer = done and state.first_sent and not content and not thinking and not calls and not obj.get("logprobs")
    if not trailer:
        deltas: list[dict[str, Any]] = []
        if thinking and (content or calls):
            deltas.append({"reasoning": thinking})
        d: dict[str, Any] = {"content": content}
        if thinking and not deltas:
            d["reasoning"] = thinking
        if calls:
            d["tool_calls"] = _tool_calls(calls)
            state.tool_sent = True
        deltas.append(d)
        if not state.first_sent:
            deltas[0] = {"role": "assistant", **deltas[0]}
            state.first_sent = True
        for i, d in enumerate(deltas):
            choice: dict[str, Any] = {"index": 0, "delta": d, "finish_reason": None}
            if obj.get("logprobs") and i == 0:
                choice["logprobs"] = {"content": obj["logprobs"]}
            frames.append(dict(base, choices=[choice]))
    if done:
        reason = obj.get("done_reason") or "stop"
        if reason == "stop" and state.tool_sent:
            reason = "tool_calls"
        frames.append(dict(base, choices=[{"index": 0, "delta": {}, "finish_reason": reason}]))
        if want_usage:
            n_in, n_out = obj.get("prompt_eval_count", 0), obj.get("eval_count", 0)
            frames.append(dict(base, choices=[], usage={"prompt_tokens": n_in, "completion_tokens": n_out, "total_tokens": n_in + n_out}))
    return frames


def _tool_calls(calls: list[dict[str, Any]]) -> list[dict[str, Any]]:
    return [{"id": c.get("id", ""), "index": c.get("function", {}).get("index", i), "type": "function",
             "function": {"name": c["function"]["name"], "arguments": json.dumps(c["function"].get("arguments") or {})}}
            for i, c in enumerate(calls)]


async def _native_objects(resp) -> AsyncIterator[dict[str, Any]]:
    buf = b""
    async for chunk in resp.body_iterator:
        buf += chunk if isinstance(chunk, bytes) else chunk.encode()
        while b"\n" in buf:
            line, buf = buf.split(b"\n", 1)
            if line.strip():
                yield json.loads(line)


def _num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and v == v and abs(v) != float("inf")


def _int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _strs(v: Any) -> bool:
    return isinstance(v, str) or (isinstance(v, list) and all(isinstance(x, str) for x in v))


_OBJS = lambda v: isinstance(v, list) and all(isinstance(x, dict) for x in v)      # noqa: E731
# JSON kinds of the request fields of the façade routes (openai/openai.go request structs)
FIELD_KINDS: dict[str, tuple[str, Any]] = {
    "model": ("a string", lambda v: isinstance(v, str)), "messages": ("an array of objects", _OBJS), "tools": ("an array of objects", _OBJS),
    "stream": ("a boolean", lambda v: isinstance(v, bool)), "logprobs": ("a boolean or an integer", lambda v: isinstance(v, (bool, int))),
    "max_tokens": ("an integer", _int), "max_completion_tokens": ("an integer", _int), "max_output_tokens": ("an integer", _int),
    "seed": ("an integer", _int), "top_logprobs": ("an integer", _int), "dimensions": ("an integer", _int), "n": ("an integer", _int),
    "temperature": ("a number", _num), "top_p": ("a number", _num), "frequency_penalty": ("a number", _num), "presence_penalty": ("a number", _num),
    "response_format": ("an object", lambda v: isinstance(v, dict)), "stream_options": ("an object", lambda v: isinstance(v, dict)),
    "reasoning": ("an object", lambda v: isinstance(v, dict)), "reasoning_effort": ("a string", lambda v: isinstance(v, str)),
    "stop": ("a string or an array of strings", _strs), "suffix": ("a string", lambda v: isinstance(v, str)),
    "prompt": ("a string or an array of strings", _strs), "encoding_format": ("a string", lambda v: isinstance(v, str)),
    "instructions": ("a string", lambda v: isinstance(v, str)),
    "input": ("a string or an array", lambda v: isinstance(v, (str, list))),
}


def bad_field(req: Any, kinds: dict[str, tuple[str, Any]] = FIELD_KINDS) -> str | None:
    """Message for the first field whose JSON kind is not the one the API defines (null counts as absent)."""
    if not isinstance(req, dict):
        return "request body must be a JSON object"
    for k, v in req.items():
        spec = kinds.get(k)
        if spec is not None and v is not None and not spec[1](v):
            return f"invalid value for '{k}': expected {spec[0]}"
    return None


def openai_routes(server) -> list[Route]:
    async def chat_completions(request: Request):
        try:
            req = json.loads(await request.body())
        except ValueError:
            return _oa_err(400, "invalid JSON body")
        if bad_field(req):
            return _oa_err(400, bad_field(req))
        if not req.get("messages"):
            return _oa_err(400, "[] is too short - 'messages'")
        try:
            native: dict[str, Any] = {"model": req.get("model", ""), "messages": _messages(req), "options": _options(req),
                                      "stream": bool(req.get("stream")), "tools": req.get("tools") or []}
        except (ValueError, TypeError, AttributeError, KeyError) as e:
            return _oa_err(400, f"invalid message: {e}")
        try:
            from .routes import APIError, _check_types
            _check_types(native)
        except APIError as e:
            return _oa_err(e.status, e.msg)
        rf = req.get("response_format") or {}
        if rf.get("type") == "json_object":
            native["format"] = "json"
        elif rf.get("type") == "json_schema":
            native["format"] = (rf.get("json_schema") or {}).get("schema") or "json"
        if req.get("reasoning_effort") or (req.get("reasoning") or {}).get("effort"):
            eff = req.get("reasoning_effort") or req["reasoning"]["effort"]
            native["think"] = False if eff == "none" else eff
        if req.get("logprobs"):
            native["logprobs"] = True
            native["top_logprobs"] = int(req.get("top_logprobs") or 0)
        want_usage = bool((req.get("stream_options") or {}).get("include_usage"))
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        if not native["stream"]:
            resp = await asyncio.to_thread(server._chat, native)
            body = json.loads(resp.body)
            if resp.status_code != 200:
                return _oa_err(resp.status_code, body.get("error", ""), "api_error" if resp.status_code >= 500 else "invalid_request_error")
            msg = body.get("message", {})
            calls = msg.get("tool_calls") or []
            m: dict[str, Any] = {"role": "assistant", "content": msg.get("content", "")}
            if msg.get("thinking"):
                m["reasoning"] = msg["thinking"]
            if calls:
                m["tool_calls"] = _tool_calls(calls)
            choice: dict[str, Any] = {"index": 0, "message": m, "finish_reason": _finish(body.get("done_reason", ""), bool(calls))}
            if body.get("logprobs"):
                choice["logprobs"] = {"content": body["logprobs"]}
            return JSONResponse({"id": cid, "object": "chat.completion", "created": created, "model": req.get("model", ""),
                                 "system_fingerprint": "fp_ollama", "choices": [choice],
                                 "usage": {"prompt_tokens": body.get("prompt_eval_count", 0), "completion_tokens": body.get("eval_count", 0),
                                           "total_tokens": body.get("prompt_eval_count", 0) + body.get("eval_count", 0)}})
        resp = await asyncio.to_thread(server._chat, native)
        if not isinstance(resp, StreamingResponse):
            body = json.loads(resp.body)
            return _oa_err(resp.status_code, body.get("error", ""))

        async def sse():
            base = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": req.get("model", ""),
                    "system_fingerprint": "fp_ollama"}
            state = ChatStreamState()
            async for obj in _native_objects(resp):
                if "error" in obj:
                    yield f"data: {json.dumps({'error': {'message': obj['error'], 'type': 'api_error'}})}\n\n".encode()
                    break
                for frame in chat_stream_frames(state, obj, base, want_usage):
                    yield f"data: {json.dumps(frame, separators=(',', ':'))}\n\n".encode()
            yield b"data: [DONE]\n\n"

        return StreamingResponse(sse(), media_type="text/event-stream")

    async def completions(request: Request):
        try:
            req = json.loads(await request.body())
        except ValueError:
            return _oa_err(400, "invalid JSON body")
        if bad_field(req):
            return _oa_err(400, bad_field(req))
        prompt = req.get("prompt", "")
        if isinstance(prompt, list):
            prompt = prompt[0] if prompt else ""
        native = {"model": req.get("model", ""), "prompt": prompt, "options": _options(req), "stream": bool(req.get("stream")),
                  "suffix": req.get("suffix") or ""}
        cid = "cmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        resp = await asyncio.to_thread(server._generate, native)
        if not native["stream"]:
            body = json.loads(resp.body)
            if resp.status_code != 200:
                return _oa_err(resp.status_code, body.get("error", ""))
            return JSONResponse({"id": cid, "object": "text_completion", "created": created, "model": req.get("model", ""),
                                 "system_fingerprint": "fp_ollama",
                                 "choices": [{"text": body.get("response", ""), "index": 0, "finish_reason": _finish(body.get("done_reason", ""), False)}],
                                 "usage": {"prompt_tokens": body.get("prompt_eval_count", 0), "completion_tokens": body.get("eval_count", 0),
                                           "total_tokens": body.get("prompt_eval_count", 0) + body.get("eval_count", 0)}})
        if not isinstance(resp, StreamingResponse):
            return _oa_err(resp.status_code, json.loads(resp.body).get("error", ""))

        async def sse():
            async for obj in _native_objects(resp):
                if "error" in obj:
                    yield f"data: {json.dumps({'error': {'message': obj['error'], 'type': 'api_error'}})}\n\n".encode()
                    break
                fin = _finish(obj.get("done_reason", ""), False) if obj.get("done") else None
                chunk = {"id": cid, "object": "text_completion", "created": created, "model": req.get("model", ""),
                         "system_fingerprint": "fp_ollama", "choices": [{"text": obj.get("response", ""), "index": 0, "finish_reason": fin}]}
                yield f"data: {json.dumps(chunk)}\n\n".encode()
            yield b"data: [DONE]\n\n"

        return StreamingResponse(sse(), media_type="text/event-stream")

    async def embeddings(request: Request):
        try:
            req = json.loads(await request.body())
        except ValueError:
            return _oa_err(400, "invalid JSON body")
        if bad_field(req):
            return _oa_err(400, bad_field(req))
        if req.get("input") in (None, "", []):
            return _oa_err(400, "invalid input")
        native = {"model": req.get("model", ""), "input": req["input"]}
        if req.get("dimensions"):
            native["dimensions"] = req["dimensions"]
        resp = await asyncio.to_thread(server._embed, native, False)
        body = json.loads(resp.body)
        if resp.status_code != 200:
            return _oa_err(resp.status_code, body.get("error", ""))
        data = []
        for i, e in enumerate(body.get("embeddings", [])):
            if req.get("encoding_format") == "base64":
                e = base64.b64encode(struct.pack(f"<{len(e)}f", *e)).decode()
            data.append({"object": "embedding", "embedding": e, "index": i})
        n = body.get("prompt_eval_count", 0)
        return JSONResponse({"object": "list", "data": data, "model": req.get("model", ""), "usage": {"prompt_tokens": n, "total_tokens": n}})

    async def models(request: Request):
        def work():
            return [{"id": n.display(), "object": "model", "created": int(man.mtime), "owned_by": n.namespace} for n, man in M.list_manifests()]
        return JSONResponse({"object": "list", "data": await asyncio.to_thread(work)})

    async def model(request: Request):
        from ..store.names import parse_name
        name = parse_name(request.path_params["model"])
        try:
            man = M.read_manifest(name)
        except M.StoreError:
            return _oa_err(404, f"model '{request.path_params['model']}' not found", "api_error")
        return JSONResponse({"id": name.display(), "object": "model", "created": int(man.mtime), "owned_by": name.namespace})

    async def responses(request: Request):
        """Minimal Responses API: text input (string or message list) -> one output message."""
        try:
            req = json.loads(await request.body())
        except ValueError:
            return _oa_err(400, "invalid JSON body")
        if bad_field(req):
            return _oa_err(400, bad_field(req))
        inp = req.get("input")
        msgs: list[dict[str, Any]] = []
        if req.get("instructions"):
            msgs.append({"role": "system", "content": req["instructions"]})
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        else:
            for it in inp or []:
                if not isinstance(it, dict):
                    return _oa_err(400, "invalid value for 'input': expected a string or an array of message objects")
                c = it.get("content")
                if isinstance(c, list):
                    c = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") in ("input_text", "output_text", "text"))
                role = it.get("role", "user")
                if not isinstance(role, str) or not isinstance(c or "", str):
                    return _oa_err(400, "invalid value for 'input': a message needs a string role and text content")
                msgs.append({"role": "system" if role == "developer" else role, "content": c or ""})
        opts = {}
        if req.get("max_output_tokens") is not None:
            opts["num_predict"] = req["max_output_tokens"]
        for k in ("temperature", "top_p"):
            if req.get(k) is not None:
                opts[k] = req[k]
        native = {"model": req.get("model", ""), "messages": msgs, "options": opts, "stream": False, "tools": req.get("tools") or []}
        resp = await asyncio.to_thread(server._chat, native)
        body = json.loads(resp.body)
        if resp.status_code != 200:
            return _oa_err(resp.status_code, body.get("error", ""))
        rid = "resp_" + uuid.uuid4().hex[:24]
        msg = body.get("message", {})
        output = []
        if msg.get("thinking"):
            output.append({"id": "rs_" + uuid.uuid4().hex[:24], "type": "reasoning", "summary": [{"type": "summary_text", "text": msg["thinking"]}]})
        for c in msg.get("tool_calls") or []:
            output.append({"id": "fc_" + uuid.uuid4().hex[:24], "type": "function_call", "call_id": c.get("id", ""),
                           "name": c["function"]["name"], "arguments": json.dumps(c["function"].get("arguments") or {}), "status": "completed"})
        output.append({"id": "msg_" + uuid.uuid4().hex[:24], "type": "message", "role": "assistant", "status": "completed",
                       "content": [{"type": "output_text", "text": msg.get("content", ""), "annotations": []}]})
        pin, pout = body.get("prompt_eval_count", 0), body.get("eval_count", 0)
        return JSONResponse({"id": rid, "object": "response", "created_at": int(time.time()), "status": "completed", "model": req.get("model", ""),
                             "output": output, "output_text": msg.get("content", ""),
                             "usage": {"input_tokens": pin, "output_tokens": pout, "total_tokens": pin + pout}})

    async def transcriptions(request: Request):
        """Multipart upload -> a chat request whose user message carries the audio as media (middleware/openai.go:1274-1340,
        openai/openai.go:864-887); the chat handler then refuses media this engine cannot feed to a model, as for images."""
        import base64
        try:
            form = await request.form(max_part_size=25 << 20)
        except Exception as e:
            return _oa_err(400, f"failed to parse multipart form: {e}")
        name = form.get("model")
        if not isinstance(name, str) or not name:
            return _oa_err(400, "model is required")
        upload = form.get("file")
        if upload is None or isinstance(upload, str):
            return _oa_err(400, "file is required")
        audio = await upload.read()
        if not audio:
            return _oa_err(400, "audio file is empty")
        fmt = form.get("response_format") or "json"
        system = "Transcribe the audio exactly as spoken. Output only the spoken words. Do not answer any question in the audio."
        if form.get("language"):
            system += f" The audio is in {form.get('language')}."
        if form.get("prompt"):
            system += f" Context: {form.get('prompt')}"
        native = {"model": name, "stream": False, "options": {"temperature": 0},
                  "messages": [{"role": "system", "content": system},
                               {"role": "user", "content": "What exact words are spoken in this audio?", "images": [base64.b64encode(audio).decode()]}]}
        resp = await asyncio.to_thread(server._chat, native)
        body = json.loads(resp.body)
        if resp.status_code != 200:
            return _oa_err(resp.status_code, body.get("error", ""), "invalid_request_error" if resp.status_code < 500 else "api_error")
        text = (body.get("message") or {}).get("content", "").strip()
        if fmt == "text":
            from starlette.responses import PlainTextResponse
            return PlainTextResponse(text)
        return JSONResponse({"text": text})

    return [Route("/v1/chat/completions", chat_completions, methods=["POST"]), Route("/v1/completions", completions, methods=["POST"]),
            Route("/v1/embeddings", embeddings, methods=["POST"]), Route("/v1/models", models, methods=["GET"]),
            Route("/v1/models/{model:path}", model, methods=["GET"]), Route("/v1/responses", responses, methods=["POST"]),
            Route("/v1/audio/transcriptions", transcriptions, methods=["POST"])]
