"""Anthropic-compatible ``/v1/messages`` route (request / response rewriting around the native chat handler;
the reference registers the same façade at server/routes.go:1926 with conversions in anthropic/)."""
from __future__ import annotations

import asyncio
import json
import uuid
from typing import Any

from starlette.requests import Request
from starlette.responses import JSONResponse, StreamingResponse
from starlette.routing import Route


def _err(status: int, msg: str, typ: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"type": "error", "error": {"type": typ, "message": msg}}, status_code=status)


def _text(content: Any) -> str:
    if isinstance(content, str):
        return content
    return "".join(b.get("text", "") for b in content or [] if b.get("type") == "text")


def _to_native(req: dict[str, Any]) -> dict[str, Any]:
    msgs: list[dict[str, Any]] = []
    if req.get("system"):
        msgs.append({"role": "system", "content": _text(req["system"])})
    for m in req.get("messages") or []:
        content = m.get("content")
        if isinstance(content, list):
            calls, results, texts, images = [], [], [], []
            for b in content:
                t = b.get("type")
                if t == "text":
                    texts.append(b.get("text", ""))
                elif t == "tool_use":
                    calls.append({"id": b.get("id", ""), "function": {"name": b.get("name", ""), "arguments": b.get("input") or {}}})
                elif t == "tool_result":
                    results.append({"role": "tool", "content": _text(b.get("content")), "tool_call_id": b.get("tool_use_id", "")})
                elif t == "image" and (b.get("source") or {}).get("type") == "base64":
                    images.append(b["source"].get("data", ""))
            if texts or calls or images:
                d: dict[str, Any] = {"role": m.get("role", "user"), "content": "".join(texts)}
                if calls:
                    d["tool_calls"] = calls
                if images:
                    d["images"] = images
                msgs.append(d)
            msgs.extend(results)
        else:
            msgs.append({"role": m.get("role", "user"), "content": content or ""})
    opts: dict[str, Any] = {"num_predict": req.get("max_tokens", -1)}
    for k in ("temperature", "top_p", "top_k"):
        if req.get(k) is not None:
            opts[k] = req[k]
    if req.get("stop_sequences"):
        opts["stop"] = req["stop_sequences"]
    tools = [{"type": "function", "function": {"name": t.get("name", ""), "description": t.get("description", ""),
                                                "parameters": t.get("input_schema") or {}}} for t in req.get("tools") or []]
    native: dict[str, Any] = {"model": req.get("model", ""), "messages": msgs, "options": opts, "tools": tools, "stream": bool(req.get("stream"))}
    th = req.get("thinking") or {}
    if th.get("type") == "enabled":
        native["think"] = True
    elif th.get("type") == "disabled":
        native["think"] = False
    return native


def _stop_reason(done_reason: str, has_tools: bool) -> str:
    return "tool_use" if has_tools else ("max_tokens" if done_reason == "length" else "end_turn")


def anthropic_routes(server) -> list[Route]:
    from .openai import FIELD_KINDS, _int, _native_objects, _num, _strs, bad_field
    from .routes import APIError
    from .routes import _check_types as check_native
    _KINDS = {**FIELD_KINDS, "system": ("a string or an array of text blocks", lambda v: isinstance(v, (str, list))),
              "stop_sequences": ("an array of strings", lambda v: isinstance(v, list) and _strs(v)),
              "thinking": ("an object", lambda v: isinstance(v, dict)), "top_k": ("an integer", _int), "temperature": ("a number", _num)}

    async def messages(request: Request):
        try:
            req = json.loads(await request.body())
        except ValueError:
            return _err(400, "invalid JSON body")
        bad = bad_field(req, _KINDS)
        if bad:
            return _err(400, bad)
        if not req.get("model"):
            return _err(400, "model is required")
        if not req.get("max_tokens"):
            return _err(400, "max_tokens is required")
        try:
            native = _to_native(req)
            check_native(native)
        except (TypeError, AttributeError, KeyError, ValueError) as e:       # content blocks of the wrong shape
            return _err(400, f"invalid request: {e}")
        except APIError as e:
            return _err(e.status, e.msg)
        mid = "msg_" + uuid.uuid4().hex[:24]
        resp = await asyncio.to_thread(server._chat, native)
        if not native["stream"]:
            body = json.loads(resp.body)
            if resp.status_code != 200:
                return _err(resp.status_code, body.get("error", ""), "not_found_error" if resp.status_code == 404 else "api_error")
            msg = body.get("message", {})
            content: list[dict[str, Any]] = []
            if msg.get("thinking"):
                content.append({"type": "thinking", "thinking": msg["thinking"], "signature": ""})
            if msg.get("content"):
                content.append({"type": "text", "text": msg["content"]})
            for c in msg.get("tool_calls") or []:
                content.append({"type": "tool_use", "id": c.get("id", ""), "name": c["function"]["name"], "input": c["function"].get("arguments") or {}})
            return JSONResponse({"id": mid, "type": "message", "role": "assistant", "model": req["model"], "content": content,
                                 "stop_reason": _stop_reason(body.get("done_reason", ""), bool(msg.get("tool_calls"))), "stop_sequence": None,
                                 "usage": {"input_tokens": body.get("prompt_eval_count", 0), "output_tokens": body.get("eval_count", 0)}})
        if not isinstance(resp, StreamingResponse):
            return _err(resp.status_code, json.loads(resp.body).get("error", ""), "api_error")

        async def sse():
            def ev(name: str, data: dict[str, Any]) -> bytes:
                return f"event: {name}\ndata: {json.dumps(data)}\n\n".encode()

            yield ev("message_start", {"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "model": req["model"],
                                                                           "content": [], "stop_reason": None, "stop_sequence": None,
                                                                           "usage": {"input_tokens": 0, "output_tokens": 0}}})
            idx, open_kind, saw_tools = -1, "", False
            async for obj in _native_objects(resp):
                if "error" in obj:
                    yield ev("error", {"type": "error", "error": {"type": "api_error", "message": obj["error"]}})
                    return
                msg = obj.get("message", {})
                for kind, text in (("thinking", msg.get("thinking", "")), ("text", msg.get("content", ""))):
                    if not text:
                        continue
                    if open_kind != kind:
                        if open_kind:
                            yield ev("content_block_stop", {"type": "content_block_stop", "index": idx})
                        idx += 1
                        open_kind = kind
                        block = {"type": "thinking", "thinking": ""} if kind == "thinking" else {"type": "text", "text": ""}
                        yield ev("content_block_start", {"type": "content_block_start", "index": idx, "content_block": block})
                    delta = {"type": "thinking_delta", "thinking": text} if kind == "thinking" else {"type": "text_delta", "text": text}
                    yield ev("content_block_delta", {"type": "content_block_delta", "index": idx, "delta": delta})
                for c in msg.get("tool_calls") or []:
                    saw_tools = True
                    if open_kind:
                        yield ev("content_block_stop", {"type": "content_block_stop", "index": idx})
                        open_kind = ""
                    idx += 1
                    yield ev("content_block_start", {"type": "content_block_start", "index": idx,
                                                     "content_block": {"type": "tool_use", "id": c.get("id", ""), "name": c["function"]["name"], "input": {}}})
                    yield ev("content_block_delta", {"type": "content_block_delta", "index": idx,
                                                     "delta": {"type": "input_json_delta", "partial_json": json.dumps(c["function"].get("arguments") or {})}})
                    yield ev("content_block_stop", {"type": "content_block_stop", "index": idx})
                if obj.get("done"):
                    if open_kind:
                        yield ev("content_block_stop", {"type": "content_block_stop", "index": idx})
                    yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": _stop_reason(obj.get("done_reason", ""), saw_tools),
                                                                                 "stop_sequence": None},
                                               "usage": {"input_tokens": obj.get("prompt_eval_count", 0), "output_tokens": obj.get("eval_count", 0)}})
                    yield ev("message_stop", {"type": "message_stop"})

        return StreamingResponse(sse(), media_type="text/event-stream")

    return [Route("/v1/messages", messages, methods=["POST"])]
