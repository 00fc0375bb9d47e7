"""`ninfer-serve`: loopback-friendly HTTP gateway (OpenAI chat / responses, Anthropic messages) over one engine.

Routes (docs/serving.md:49-61 of the reference): GET /health, GET /v1/models[/{id}], POST /v1/chat/completions,
POST /v1/responses, POST /v1/responses/input_tokens, POST /v1/responses/compact, GET|DELETE /v1/responses/{id},
GET /v1/responses/{id}/input_items, POST /v1/messages, POST /v1/messages/count_tokens.  Streaming is SSE with a
5-second keep-alive comment; a client that goes away cancels its generation.  Bearer / x-api-key
authentication (health exempt), 429 `server_overloaded`, 503 `request_queue_timeout`, JSONL request log.
Reference: src/serve/http_server.cpp:408-500, docs/serving.md:66-73, :658-705, :829-835.
"""
from __future__ import annotations

import hmac
import json
import socket
import threading
import time
from collections import OrderedDict
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, Iterator, Optional

from ..runtime.engine import RequestError, ResourceError
from . import protocols as P
from .request_log import RequestLog
from .service import GenerationService, GenRequest, GenResult

KEEPALIVE_S = 5.0
DEAD_PEER_MS = 15000   # TCP_USER_TIMEOUT on accepted connections (0 = leave the kernel default)


class _Keepalive:
    """Wraps a blocking event iterator so that the writer can emit SSE comments while the model is busy."""

    def __init__(self, it: Iterator[tuple]):
        import queue
        self.q: "queue.Queue" = queue.Queue()
        self._t = threading.Thread(target=self._pump, args=(it,), daemon=True)
        self._t.start()

    def _pump(self, it):
        try:
            for item in it:
                self.q.put(("item", item))
            self.q.put(("end", None))
        except BaseException as e:  # surfaced in the consumer thread
            self.q.put(("exc", e))

    def __iter__(self):
        import queue
        while True:
            try:
                kind, item = self.q.get(timeout=KEEPALIVE_S)
            except queue.Empty:
                yield None  # keep-alive tick
                continue
            if kind == "item":
                yield item
            elif kind == "exc":
                raise item
            else:
                return


class ServeState:
    def __init__(self, service: GenerationService, api_key: Optional[str] = None, log_path: Optional[str] = None,
                 max_body_bytes: int = 32 << 20, max_stored_responses: int = 512, max_stored_bytes: int = 256 << 20,
                 cors: bool = False, log_interval_s: float = 5.0, default_max_tokens: Optional[int] = None,
                 default_thinking: bool = True):
        self.service, self.api_key, self.max_body = service, api_key, max_body_bytes
        self.cors = bool(cors)
        self.default_max_tokens = default_max_tokens       # output limit of a request that names none
        self.default_thinking = bool(default_thinking)     # thinking mode of a request that names none
        self.max_stored_bytes = max(1, int(max_stored_bytes))
        self.stored_bytes = 0
        from .rag import DocumentStore
        self.documents = DocumentStore()       # retrieval-augmented answering (serve/rag.py)
        self.log = RequestLog(log_path, throughput_every_s=log_interval_s if log_interval_s > 0 else float("inf"))
        # local response store: bounded, the least recently used entry goes first (a stored response keeps its
        # whole message history, so an unbounded store would grow with the server's life)
        self.responses: "OrderedDict[str, dict]" = OrderedDict()
        self.max_stored_responses = max(1, int(max_stored_responses))
        self.lock = threading.Lock()
        import sys as _sys

        from .request_log import redact_argv
        eng = service.engine
        self.log.event("server_start", model=service.model_id, max_concurrent=service.max_concurrent,
                       engine={"max_context": getattr(eng, "_max_context", None), "max_pending": getattr(eng, "max_pending", None),
                               "free_lanes": eng.health().get("free_lanes")},
                       argv=redact_argv(_sys.argv))


def make_handler(state: ServeState):
    svc = state.service

    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "ninfer-fusion-b200"

        def log_message(self, fmt, *args):  # the JSONL log replaces the default stderr access log
            pass

        def setup(self):
            super().setup()
            # Dead-peer detection: unacknowledged stream bytes (the 5-second keep-alive comments included) fail the
            # connection after DEAD_PEER_MS instead of after the kernel's retransmission schedule (minutes), so a
            # client that vanished stops costing decode rounds.  Linux only; elsewhere the write error comes later.
            opt = getattr(socket, "TCP_USER_TIMEOUT", None)
            if opt is not None and DEAD_PEER_MS > 0:
                try:
                    self.connection.setsockopt(socket.IPPROTO_TCP, opt, DEAD_PEER_MS)
                except OSError:
                    pass

        # ---------------------------------------------------------------- helpers
        def _send_json(self, code: int, obj: dict, headers: Optional[dict] = None) -> None:
            data = json.dumps(obj, ensure_ascii=False).encode("utf-8")
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            for k, v in (headers or {}).items():
                self.send_header(k, v)
            self._cors_headers()
            self.end_headers()
            self.wfile.write(data)

        def _cors_headers(self) -> None:
            if state.cors:      # permissive browser access (--cors): any origin may call, the key still applies
                self.send_header("Access-Control-Allow-Origin", "*")
                self.send_header("Access-Control-Allow-Headers", "authorization, content-type, x-api-key, anthropic-version")
                self.send_header("Access-Control-Allow-Methods", "GET, POST, DELETE, OPTIONS")

        def do_OPTIONS(self):
            self.send_response(204 if state.cors else 405)
            self._cors_headers()
            self.send_header("Content-Length", "0")
            self.end_headers()

        def _error(self, code: int, message: str, etype: str = "invalid_request_error", param=None, ecode=None,
                   anthropic: bool = False) -> None:
            if anthropic:
                self._send_json(code, {"type": "error", "error": {"type": etype, "message": message}})
            else:
                self._send_json(code, {"error": {"message": message, "type": etype, "param": param, "code": ecode or etype}})

        def _authorized(self) -> bool:
            if not state.api_key:
                return True
            want = state.api_key.encode()
            auth = self.headers.get("Authorization", "")
            # constant-time comparisons: the time to a refusal must not depend on how much of the key matched
            if auth.startswith("Bearer ") and hmac.compare_digest(auth[7:].strip().encode(), want):
                return True
            return hmac.compare_digest(self.headers.get("x-api-key", "").encode(), want)

        def _body(self) -> dict:
            try:
                n = int(self.headers.get("Content-Length", "0") or 0)
            except ValueError:
                raise P.BadRequest("Content-Length is not a number") from None
            if n <= 0:
                raise P.BadRequest("request body is empty")
            if n > state.max_body:
                raise P.BadRequest("request body too large", code="request_too_large")
            try:
                obj = json.loads(self.rfile.read(n))
            except json.JSONDecodeError as e:
                raise P.BadRequest(f"body is not valid JSON: {e}") from None
            if not isinstance(obj, dict):
                raise P.BadRequest("body must be a JSON object")
            return obj

        def _stream(self, chunks: Iterator[Optional[bytes]]) -> bool:
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self._cors_headers()
            self.end_headers()
            self.close_connection = True
            try:
                for c in chunks:
                    self.wfile.write(c if c is not None else b": keep-alive\n\n")
                    self.wfile.flush()
                return True
            except (BrokenPipeError, ConnectionResetError, OSError):
                return False

        # ---------------------------------------------------------------- generation plumbing
        def _run(self, api: str, req: GenRequest, stream: bool, build, build_stream, anthropic: bool = False):
            t0 = time.time()
            gone = threading.Event()
            info = {}

            def on_start(rid, n_prompt):
                info["rid"], info["prompt_tokens"] = rid, n_prompt
                state.log.event("request_start", request_id=rid, protocol=api, stream=bool(stream), prompt_tokens=n_prompt,
                                sampler={"temperature": req.temperature, "top_p": req.top_p, "top_k": req.top_k,
                                         "seed": req.seed}, output_budget=req.max_tokens,
                                thinking=bool(getattr(req, "enable_thinking", True)), session=bool(req.session))

            def finished(res: GenResult):
                state.log.request_done(res, api, stream, speculative=getattr(res, "speculative", None))

            try:
                events = svc.stream(req, on_start=on_start, cancelled=gone.is_set)
                if not stream:
                    res = None
                    for kind, item in events:
                        if kind == "done":
                            res = item
                    finished(res)
                    if res.finish_reason == "error":
                        return self._error(500, res.error or "generation failed", "api_error", anthropic=anthropic)
                    if res.finish_reason == "timeout":
                        return self._error(503, "request_queue_timeout", "server_error", ecode="request_queue_timeout",
                                           anthropic=anthropic)
                    return self._send_json(200, build(res))

                # the first event is pulled before the 200 header goes out, so that admission errors and queue
                # time-outs still get a proper status code
                first = next(events)
                if first[0] == "done" and first[1].finish_reason in ("error", "timeout"):
                    finished(first[1])
                    if first[1].finish_reason == "timeout":
                        return self._error(503, "request_queue_timeout", "server_error", ecode="request_queue_timeout",
                                           anthropic=anthropic)
                    return self._error(500, first[1].error or "generation failed", "api_error", anthropic=anthropic)

                def all_events():
                    yield first
                    yield from events

                def tap(it):
                    for ev in it:
                        if ev[0] == "done":
                            finished(ev[1])
                        yield ev

                if not self._stream(iter(_Keepalive(build_stream(tap(all_events()))))):
                    gone.set()
                    state.log.event("request_error", request_id=info.get("rid"), protocol=api, error="client disconnected")
            except ResourceError as e:
                state.log.event("request_rejected", protocol=api, phase="prepare", message=str(e))
                if "timeout" in str(e):
                    self._error(503, str(e), "server_error", ecode="request_queue_timeout", anthropic=anthropic)
                else:
                    self._error(429, str(e), "overloaded_error" if anthropic else "server_overloaded",
                                ecode="server_overloaded", anthropic=anthropic)
            except (RequestError, P.BadRequest) as e:
                state.log.event("request_rejected", protocol=api, phase="prepare", message=str(e))
                self._error(400, str(e), "invalid_request_error", getattr(e, "param", None), anthropic=anthropic)
            finally:
                h = svc.engine.health()
                state.log.throughput(svc.engine.stats.as_dict(), {"running": h.get("active"), "waiting": h.get("pending"),
                                                                  "free_lanes": h.get("free_lanes")})

        # ---------------------------------------------------------------- routes
        def do_GET(self):
            path = self.path.split("?", 1)[0].rstrip("/") or "/"
            if path == "/health":
                return self._send_json(200, svc.health())
            if path in ("/", "/console", "/rag"):
                # the browser pages: static, without data of their own, so they need no key (their calls do)
                from .console import page_bytes
                from .rag import page_bytes as rag_page
                data = rag_page() if path == "/rag" else page_bytes()
                self.send_response(200)
                self.send_header("Content-Type", "text/html; charset=utf-8")
                self.send_header("Content-Length", str(len(data)))
                self.send_header("Cache-Control", "no-store")
                self.end_headers()
                self.wfile.write(data)
                return
            if not self._authorized():
                return self._error(401, "invalid API key", "authentication_error")
            model_obj = {"id": svc.model_id, "object": "model", "created": int(svc.started), "owned_by": "ninfer-fusion-b200"}
            if path == "/v1/models":
                return self._send_json(200, {"object": "list", "data": [model_obj]})
            if path.startswith("/v1/models/"):
                if path[len("/v1/models/"):] == svc.model_id:
                    return self._send_json(200, model_obj)
                return self._error(404, "model not found", "not_found_error")
            if path == "/v1/rag/documents":
                return self._send_json(200, {"object": "list", "data": state.documents.list()})
            if path.startswith("/v1/responses/"):
                rest = path[len("/v1/responses/"):]
                rid, _, tail = rest.partition("/")
                with state.lock:
                    obj = state.responses.get(rid)
                    if obj is not None:
                        state.responses.move_to_end(rid)   # recently read = recently used
                if obj is None:
                    return self._error(404, f"response '{rid}' not found", "not_found_error")
                if tail == "input_items":
                    items = [{"type": "message", "role": m.get("role"), "content": m.get("content")} for m in obj["_input"]]
                    return self._send_json(200, {"object": "list", "data": items, "has_more": False})
                if tail == "":
                    return self._send_json(200, {k: v for k, v in obj.items() if not k.startswith("_")})
            return self._error(404, f"no route for GET {path}", "not_found_error")

        def do_DELETE(self):
            path = self.path.split("?", 1)[0].rstrip("/")
            if not self._authorized():
                return self._error(401, "invalid API key", "authentication_error")
            if path.startswith("/v1/responses/"):
                rid = path[len("/v1/responses/"):]
                with state.lock:
                    gone = state.responses.pop(rid, None)
                    found = gone is not None
                    if found:
                        state.stored_bytes -= gone.get("_bytes", 0)
                if found:
                    return self._send_json(200, {"id": rid, "object": "response", "deleted": True})
                return self._error(404, f"response '{rid}' not found", "not_found_error")
            if path.startswith("/v1/rag/documents/"):
                did = path[len("/v1/rag/documents/"):]
                if state.documents.remove(did):
                    return self._send_json(200, {"id": did, "object": "rag.document", "deleted": True})
                return self._error(404, f"document '{did}' not found", "not_found_error")
            return self._error(404, f"no route for DELETE {path}", "not_found_error")

        def do_POST(self):
            path = self.path.split("?", 1)[0].rstrip("/")
            anthropic = path.startswith("/v1/messages")
            if not self._authorized():
                return self._error(401, "invalid API key", "authentication_error", anthropic=anthropic)
            try:
                body = self._body()
                if state.default_max_tokens and not anthropic:
                    key = "max_output_tokens" if path.startswith("/v1/responses") else "max_tokens"
                    if body.get(key) is None and body.get("max_completion_tokens") is None:
                        body[key] = int(state.default_max_tokens)
                if not state.default_thinking and path == "/v1/chat/completions" and "enable_thinking" not in body \
                        and "enable_thinking" not in (body.get("chat_template_kwargs") or {}):
                    body["enable_thinking"] = False
                if path == "/v1/chat/completions":
                    req, o = P.parse_openai_chat(body)
                    return self._run("openai_chat", req, o["stream"], lambda r: P.openai_chat_response(r, svc.model_id),
                                     lambda ev: P.openai_chat_stream(ev, svc.model_id, o["include_usage"]))
                if path == "/v1/responses":
                    with state.lock:
                        snapshot = dict(state.responses)
                    req, o = P.parse_openai_responses(body, snapshot)

                    def remember(obj: dict, res: GenResult):
                        if o["store"]:
                            rec = dict(obj)
                            rec["_input"] = o["messages"]
                            rec["_messages"] = o["messages"] + [{"role": "assistant", "content": res.content}]
                            rec["_bytes"] = len(json.dumps(rec, ensure_ascii=False))
                            with state.lock:
                                old = state.responses.pop(obj["id"], None)
                                if old is not None:
                                    state.stored_bytes -= old.get("_bytes", 0)
                                state.responses[obj["id"]] = rec
                                state.stored_bytes += rec["_bytes"]
                                # two bounds: records and bytes (a stored response keeps its whole message history)
                                while len(state.responses) > 1 and (len(state.responses) > state.max_stored_responses
                                                                    or state.stored_bytes > state.max_stored_bytes):
                                    _, gone = state.responses.popitem(last=False)
                                    state.stored_bytes -= gone.get("_bytes", 0)

                    def build(res: GenResult):
                        obj = P.openai_responses_object(res, svc.model_id)
                        remember(obj, res)
                        return obj
                    return self._run("openai_responses", req, o["stream"], build,
                                     lambda ev: P.openai_responses_stream(ev, svc.model_id, remember))
                if path == "/v1/rag/documents":
                    try:
                        return self._send_json(200, dict(state.documents.add(body.get("title", ""), body.get("text")), object="rag.document"))
                    except ValueError as e:
                        raise P.BadRequest(str(e), "text") from None
                if path == "/v1/rag/query":
                    query = body.get("query")
                    if not isinstance(query, str) or not query.strip():
                        raise P.BadRequest("query must be a non-empty string", "query")
                    hits = state.documents.retrieve(query, int(body.get("top_k", 4)))
                    msgs, sources = state.documents.build_messages(query, hits)
                    chat = {k: body[k] for k in ("max_tokens", "temperature", "top_p", "top_k_sampling", "seed", "thinking_budget")
                            if k in body}
                    chat["messages"] = msgs
                    chat.setdefault("enable_thinking", bool(body.get("enable_thinking", False)))
                    req, _ = P.parse_openai_chat(chat)
                    return self._run("rag_query", req, False,
                                     lambda r: {"object": "rag.answer", "answer": r.content, "sources": sources,
                                                "usage": P._usage_openai(r), "finish_reason": r.finish_reason},
                                     lambda ev: iter(()))
                if path == "/v1/responses/input_tokens":
                    req, _ = P.parse_openai_responses(body, dict(state.responses))
                    return self._send_json(200, {"object": "response.input_tokens", "input_tokens": svc.count_tokens(req)})
                if path == "/v1/responses/compact":
                    # keeps the system prompt and the most recent turns that fit the requested budget
                    msgs = P.responses_input_to_messages(body, dict(state.responses))
                    budget = int(body.get("max_input_tokens") or 4096)
                    kept, used = [], 0
                    head = [m for m in msgs[:1] if m.get("role") == "system"]
                    for m in reversed(msgs[len(head):]):
                        n = svc.count_tokens(GenRequest(messages=[m]))
                        if used + n > budget and kept:
                            break
                        kept.append(m)
                        used += n
                    items = [{"type": "message", "role": m["role"], "content": m.get("content")} for m in head + kept[::-1]]
                    return self._send_json(200, {"object": "response.compaction", "output": items, "input_tokens": used})
                if path == "/v1/messages":
                    req, o = P.parse_anthropic_messages(body)
                    hint = svc.count_tokens(req) if o["stream"] else 0
                    return self._run("anthropic_messages", req, o["stream"],
                                     lambda r: P.anthropic_message_response(r, svc.model_id),
                                     lambda ev: P.anthropic_stream(ev, svc.model_id, hint), anthropic=True)
                if path == "/v1/messages/count_tokens":
                    body.setdefault("max_tokens", 1)
                    req, _ = P.parse_anthropic_messages(body)
                    return self._send_json(200, {"input_tokens": svc.count_tokens(req)})
                return self._error(404, f"no route for POST {path}", "not_found_error", anthropic=anthropic)
            except P.BadRequest as e:
                state.log.event("request_rejected", protocol=path, phase="prepare", message=str(e))
                return self._error(404 if e.code == "not_found" else 400, str(e), "invalid_request_error", e.param,
                                   e.code, anthropic=anthropic)

    return Handler


def serve(service: GenerationService, host: str = "127.0.0.1", port: int = 8080, api_key: Optional[str] = None,
          log_path: Optional[str] = None, max_stored_responses: int = 512, **state_options) -> ThreadingHTTPServer:
    """Builds the server (not yet serving): call `.serve_forever()` or run it in a thread; `.shutdown()` stops it.
    `state_options`: ServeState's further settings (max_body_bytes, max_stored_bytes, cors, log_interval_s,
    default_max_tokens, default_thinking)."""
    state = ServeState(service, api_key, log_path, max_stored_responses=max_stored_responses, **state_options)
    httpd = ThreadingHTTPServer((host, port), make_handler(state))
    httpd.daemon_threads = True
    httpd.state = state  # type: ignore[attr-defined]
    return httpd
