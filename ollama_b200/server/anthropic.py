"""Anthropic-compatible ``/v1/messages`` route (request / response rewriting around the native chat handler;
the reference registers the same façade at server/routes.go:1926 with conversions in anthropic/).

Server tools: a tool of type ``web_search_*`` is offered to the model as the function ``web_search(query)`` and its calls
are answered here, not by the client (middleware/anthropic.go:88-372): the query goes to the search service, the results go
back to the model as a tool message, and this repeats up to three times before the answer is returned with one
``server_tool_use`` + ``web_search_tool_result`` pair per search in front of the model's own blocks.  The search function
is a server attribute (``server.web_search``), so deployments without the cloud service can plug in their own; the built-in
one posts a signed request to the service and refuses when cloud features are off.
"""
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
    tools, server_tools = split_server_tools(req.get("tools"))
    native: dict[str, Any] = {"model": req.get("model", ""), "messages": msgs, "options": opts, "tools": tools, "stream": bool(req.get("stream"))}
    if server_tools:
        native["_server_tools"] = True
    th = req.get("thinking") or {}
    if th.get("type") == "enabled":
        native["think"] = True
    elif th.get("type") == "disabled":
        native["think"] = False
    return native


MAX_WEB_SEARCHES = 3
WEB_SEARCH_TOOL = {"type": "function", "function": {
    "name": "web_search", "description": "Search the web for current information. Use this to find up-to-date information about any topic.",
    "parameters": {"type": "object", "required": ["query"], "properties": {"query": {"type": "string", "description": "The search query to look up on the web"}}}}}


def split_server_tools(tools: list[dict[str, Any]] | None) -> tuple[list[dict[str, Any]], bool]:
    """Client tools in the request's order, the web-search server tool (if asked for) as a function; a client tool that
    happens to be called ``web_search`` gives way to the server tool."""
    tools = tools or []
    wants_search = any(str(t.get("type", "")).startswith("web_search") for t in tools)
    out = []
    for t in tools:
        if str(t.get("type", "")).startswith("web_search"):
            if WEB_SEARCH_TOOL not in out:
                out.append(WEB_SEARCH_TOOL)
        elif not (wants_search and t.get("name") == "web_search"):
            out.append({"type": "function", "function": {"name": t.get("name", ""), "description": t.get("description", ""),
                                                          "parameters": t.get("input_schema") or {}}})
    return out, wants_search


def cloud_web_search(query: str, max_results: int = 5) -> list[dict[str, str]]:
    """The hosted search service (anthropic/anthropic.go:1189-1262): a POST signed with this machine's key."""
    import time
    import urllib.request

    from .. import auth, envconfig
    if envconfig.no_cloud():
        raise RuntimeError("web search is unavailable: cloud features are disabled")
    path = f"/api/web_search?ts={int(time.time())}"
    body = json.dumps({"query": query, "max_results": max(1, min(int(max_results or 5), 10))}).encode()
    req = urllib.request.Request("https://ollama.com" + path, data=body, method="POST", headers={"Content-Type": "application/json"})
    try:
        req.add_header("Authorization", "Bearer " + auth.sign(f"POST,{path}".encode()))
    except Exception:                                # no key pair: the service will answer 401, which is reported below
        pass
    with urllib.request.urlopen(req, timeout=15) as r:
        return list(json.load(r).get("results") or [])


def _search_call(calls: list[dict[str, Any]] | None) -> dict[str, Any] | None:
    return next((c for c in calls or [] if (c.get("function") or {}).get("name") == "web_search"), None)


def _result_text(results: list[dict[str, str]]) -> str:
    return "".join(f"Title: {r.get('title', '')}\nURL: {r.get('url', '')}\n" + (f"Content: {r['content']}\n" if r.get("content") else "") + "\n"
                   for r in results)


def _blocks(msg: dict[str, Any]) -> list[dict[str, Any]]:
    content: list[dict[str, Any]] = []
    if msg.get("thinking"):
        content.append({"type": "thinking", "thinking": msg["thinking"], "signature": ""})
    if msg.get("content"):
        content.append({"type": "text", "text": msg["content"]})
    for c in msg.get("tool_calls") or []:
        content.append({"type": "tool_use", "id": c.get("id", ""), "name": c["function"]["name"], "input": c["function"].get("arguments") or {}})
    return content


def run_web_search_loop(chat, native: dict[str, Any], first: dict[str, Any], search, mid: str, model: str) -> dict[str, Any]:
    """``chat(request)`` -> the body of a non-streaming native chat; ``first`` is the body that contained the first
    ``web_search`` call.  Returns the Anthropic message."""
    base = "srvtoolu_" + mid.removeprefix("msg_")
    usage = {"input_tokens": first.get("prompt_eval_count", 0), "output_tokens": first.get("eval_count", 0)}
    messages = list(native["messages"])
    served: list[dict[str, Any]] = []

    def pair(n: int, query: str, result: Any) -> None:
        tid = base if n <= 1 else f"{base}_{n}"
        served.append({"type": "server_tool_use", "id": tid, "name": "web_search", "input": {"query": query}})
        served.append({"type": "web_search_tool_result", "tool_use_id": tid, "content": result})

    def failed(n: int, query: str, code: str) -> dict[str, Any]:
        pair(n, query, {"type": "web_search_tool_result_error", "error_code": code})
        return {"id": mid, "type": "message", "role": "assistant", "model": model, "content": served, "stop_reason": "end_turn",
                "stop_sequence": None, "usage": usage}

    body = first
    for n in range(1, MAX_WEB_SEARCHES + 1):
        msg = body.get("message", {})
        call = _search_call(msg.get("tool_calls"))
        query = str(((call or {}).get("function") or {}).get("arguments", {}).get("query") or "").strip()
        if not query:
            return failed(n, "", "invalid_request")
        try:
            results = search(query, 5)
        except Exception:
            return failed(n, query, "unavailable")
        pair(n, query, [{"type": "web_search_result", "url": r.get("url", ""), "title": r.get("title", "")} for r in results])
        messages.append({"role": "assistant", "content": msg.get("content", ""), "thinking": msg.get("thinking", ""), "tool_calls": [call]})
        messages.append({"role": "tool", "content": _result_text(results), "tool_call_id": call.get("id", "")})
        try:
            body = chat({**native, "messages": messages, "stream": False})
        except Exception:
            return failed(n, query, "api_error")
        usage["input_tokens"] += body.get("prompt_eval_count", 0)
        usage["output_tokens"] += body.get("eval_count", 0)
        msg = body.get("message", {})
        if _search_call(msg.get("tool_calls")) is None:
            return {"id": mid, "type": "message", "role": "assistant", "model": model, "content": served + _blocks(msg),
                    "stop_reason": _stop_reason(body.get("done_reason", ""), bool(msg.get("tool_calls"))), "stop_sequence": None, "usage": usage}
    last = _search_call(body.get("message", {}).get("tool_calls")) or {}
    return failed(MAX_WEB_SEARCHES + 1, str((last.get("function") or {}).get("arguments", {}).get("query") or ""), "max_uses_exceeded")


def message_events(message: dict[str, Any]) -> list[tuple[str, dict[str, Any]]]:
    """A finished message as the event sequence of a stream: every block opens, delivers its whole payload, closes."""
    shell = {**message, "content": [], "stop_reason": None, "usage": {"input_tokens": message["usage"]["input_tokens"], "output_tokens": 0}}
    ev: list[tuple[str, dict[str, Any]]] = [("message_start", {"type": "message_start", "message": shell})]
    for i, b in enumerate(message["content"]):
        kind = b["type"]
        start = {"text": {"type": "text", "text": ""}, "thinking": {"type": "thinking", "thinking": ""},
                 "tool_use": {**b, "input": {}}, "server_tool_use": {**b, "input": {}}}.get(kind, b)
        ev.append(("content_block_start", {"type": "content_block_start", "index": i, "content_block": start}))
        delta = ({"type": "text_delta", "text": b["text"]} if kind == "text" else {"type": "thinking_delta", "thinking": b["thinking"]} if kind == "thinking"
                 else {"type": "input_json_delta", "partial_json": json.dumps(b.get("input") or {})} if kind in ("tool_use", "server_tool_use") else None)
        if delta is not None:
            ev.append(("content_block_delta", {"type": "content_block_delta", "index": i, "delta": delta}))
        ev.append(("content_block_stop", {"type": "content_block_stop", "index": i}))
    ev.append(("message_delta", {"type": "message_delta", "delta": {"stop_reason": message["stop_reason"], "stop_sequence": None},
                                 "usage": message["usage"]}))
    ev.append(("message_stop", {"type": "message_stop"}))
    return ev


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
        if native.pop("_server_tools", False):
            # the searches happen between model turns, so the turns run unstreamed and a streaming client gets the finished
            # message as one burst of events
            def chat(request: dict[str, Any]) -> dict[str, Any]:
                r = server._chat(request)
                out = json.loads(r.body)
                if r.status_code != 200:
                    raise APIError(r.status_code, out.get("error", ""))
                return out

            def whole() -> dict[str, Any]:
                first = chat({**native, "stream": False})
                msg = first.get("message", {})
                if _search_call(msg.get("tool_calls")) is None:
                    return {"id": mid, "type": "message", "role": "assistant", "model": req["model"], "content": _blocks(msg),
                            "stop_reason": _stop_reason(first.get("done_reason", ""), bool(msg.get("tool_calls"))), "stop_sequence": None,
                            "usage": {"input_tokens": first.get("prompt_eval_count", 0), "output_tokens": first.get("eval_count", 0)}}
                return run_web_search_loop(chat, native, first, getattr(server, "web_search", None) or cloud_web_search, mid, req["model"])

            try:
                message = await asyncio.to_thread(whole)
            except APIError as e:
                return _err(e.status, e.msg, "not_found_error" if e.status == 404 else "api_error")
            if not req.get("stream"):
                return JSONResponse(message)

            async def burst():
                for name, data in message_events(message):
                    yield f"event: {name}\ndata: {json.dumps(data)}\n\n".encode()
            return StreamingResponse(burst(), media_type="text/event-stream")
        resp = await asyncio.to_thread(server._chat, native)
        if not native["stream"]:
            body = json.loads(resp.body)
            if resp.status_code != 200:
                return _err(resp.status_code, body.get("error", ""), "not_found_error" if resp.status_code == 404 else "api_error")
            msg = body.get("message", {})
            content = _blocks(msg)
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
