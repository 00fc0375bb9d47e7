"""Protocol translators: OpenAI chat completions, OpenAI responses and Anthropic messages <-> GenRequest/GenResult.

Each gateway has three parts: request parsing (closed member sets: unknown knobs that change semantics are
rejected, cosmetic ones ignored), the non-streaming response body, and the SSE event sequence.  Shapes follow
the reference's gateways (src/serve/openai_chat_*.cpp, openai_responses_*.cpp, anthropic_messages_*.cpp;
route table docs/serving.md:49-61).
"""
from __future__ import annotations

import json
import time
import uuid
from typing import Dict, Iterator, List, Optional, Tuple

from ..frontend.chat import ParsedDelta
from .service import GenRequest, GenResult


class BadRequest(ValueError):
    def __init__(self, message: str, param: Optional[str] = None, code: str = "invalid_request_error"):
        super().__init__(message)
        self.param, self.code = param, code


def _stops(v) -> List[str]:
    if v is None:
        return []
    if isinstance(v, str):
        return [v]
    if isinstance(v, list) and all(isinstance(s, str) for s in v) and len(v) <= 8:
        return v
    raise BadRequest("stop must be a string or a list of up to 8 strings", "stop")


def _num(body: dict, key: str, lo: float, hi: float, cast=float):
    v = body.get(key)
    if v is None:
        return None
    try:
        v = cast(v)
    except (TypeError, ValueError):
        raise BadRequest(f"{key} must be a number", key) from None
    if not (lo <= v <= hi):
        raise BadRequest(f"{key} must be in [{lo}, {hi}]", key)
    return v


def sse(data, event: Optional[str] = None) -> bytes:
    head = f"event: {event}\n" if event else ""
    body = data if isinstance(data, str) else json.dumps(data, ensure_ascii=False, separators=(",", ":"))
    return (head + "data: " + body + "\n\n").encode("utf-8")


# =========================================================================================================
# Prompt-cache hints
# =========================================================================================================
def _openai_cache_hints(body: dict, msgs: List[dict]) -> dict:
    """OpenAI prompt caching (`prompt_cache_options`, `prompt_cache_breakpoint` on messages or content parts,
    `prompt_cache_key`, `prompt_cache_retention`) as write candidates for the shared-prefix catalogue.  The fields are
    optimisation hints: they are validated, never change the prompt, and promise no wall-clock residency."""
    out = {"cache_implicit": True, "cache_breakpoints": [], "cache_key": None, "cache_retention": None}
    po = body.get("prompt_cache_options")
    if po is not None:
        if not isinstance(po, dict) or po.get("mode", "implicit") not in ("implicit", "explicit"):
            raise BadRequest("prompt_cache_options.mode must be 'implicit' or 'explicit'", "prompt_cache_options")
        out["cache_implicit"] = po.get("mode", "implicit") == "implicit"
    key = body.get("prompt_cache_key")
    if key is not None:
        if not isinstance(key, str) or len(key) > 512:
            raise BadRequest("prompt_cache_key must be a string of at most 512 characters", "prompt_cache_key")
        out["cache_key"] = key
    ret = body.get("prompt_cache_retention")
    if ret is not None:
        if ret not in ("in_memory", "24h"):
            raise BadRequest("prompt_cache_retention must be 'in_memory' or '24h'", "prompt_cache_retention")
        out["cache_retention"] = ret

    def marked(obj) -> bool:
        bp = obj.get("prompt_cache_breakpoint") if isinstance(obj, dict) else None
        if bp is None:
            return False
        if not isinstance(bp, dict) or bp.get("mode", "explicit") != "explicit":
            raise BadRequest("prompt_cache_breakpoint.mode must be 'explicit'", "prompt_cache_breakpoint")
        return True
    for i, m in enumerate(msgs):
        parts = m.get("content") if isinstance(m.get("content"), list) else []
        if marked(m) or any(marked(p) for p in parts):
            out["cache_breakpoints"].append(i)
    return out


def _anthropic_cache_marked(obj) -> bool:
    cc = obj.get("cache_control") if isinstance(obj, dict) else None
    if cc is None:
        return False
    if not isinstance(cc, dict) or cc.get("type") != "ephemeral":
        raise BadRequest("cache_control.type must be 'ephemeral'", "cache_control")
    if cc.get("ttl") not in (None, "5m", "1h"):
        raise BadRequest("cache_control.ttl must be '5m' or '1h'", "cache_control")
    return True


# =========================================================================================================
# OpenAI chat completions
# =========================================================================================================
def _soft_max(body: dict, key: str, hard: int) -> Optional[int]:
    """Extension field: completion tokens after which the generation ends at the next syntax-safe boundary."""
    v = body.get(key)
    if v is None:
        return None
    if not isinstance(v, int) or isinstance(v, bool) or v < 1:
        raise BadRequest(f"{key} must be a positive integer", key)
    if v > hard:
        raise BadRequest(f"{key} must not exceed the hard limit ({hard})", key)
    return v


def _with_boundary(obj: dict, res: GenResult) -> dict:
    if getattr(res, "stop_boundary", None):
        obj["stop_boundary"] = res.stop_boundary       # out of band: never part of the generated text
    return obj


def parse_openai_chat(body: dict) -> Tuple[GenRequest, dict]:
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise BadRequest("messages must be a non-empty list", "messages")
    if body.get("n", 1) != 1:
        raise BadRequest("only n = 1 is supported", "n")
    rf = body.get("response_format")
    if isinstance(rf, dict) and rf.get("type") not in (None, "text"):
        raise BadRequest("structured output modes are not supported", "response_format", "unsupported_parameter")
    kw = body.get("chat_template_kwargs") or {}
    thinking = bool(kw.get("enable_thinking", body.get("enable_thinking", True)))
    tools = body.get("tools")
    if tools is not None and body.get("tool_choice") == "none":
        tools = None
    max_tokens = body.get("max_completion_tokens", body.get("max_tokens", 512))
    budget = kw.get("thinking_budget", body.get("thinking_budget"))
    if budget is not None and (not isinstance(budget, int) or isinstance(budget, bool) or budget < 1):
        raise BadRequest("thinking_budget must be a positive integer", "thinking_budget")
    req = GenRequest(messages=msgs, tools=tools, max_tokens=int(max_tokens), thinking_budget=budget,
                     temperature=_num(body, "temperature", 0.0, 2.0), top_p=_num(body, "top_p", 0.0, 1.0),
                     top_k=_num(body, "top_k", 1, 20, int), min_p=_num(body, "min_p", 0.0, 1.0),
                     presence_penalty=_num(body, "presence_penalty", -2.0, 2.0),
                     frequency_penalty=_num(body, "frequency_penalty", -2.0, 2.0),
                     seed=_num(body, "seed", 0, 2 ** 63 - 1, int), stop=_stops(body.get("stop")),
                     enable_thinking=thinking, session=body.get("user"),
                     soft_max_tokens=_soft_max(body, "soft_max_tokens", int(max_tokens)), **_openai_cache_hints(body, msgs))
    opts = {"stream": bool(body.get("stream", False)),
            "include_usage": bool((body.get("stream_options") or {}).get("include_usage", False))}
    return req, opts


def _usage_openai(res: GenResult) -> dict:
    return {"prompt_tokens": res.prompt_tokens, "completion_tokens": res.completion_tokens,
            "total_tokens": res.prompt_tokens + res.completion_tokens,
            "prompt_tokens_details": {"cached_tokens": int(getattr(res, "cached_tokens", 0) or 0)}}


def _finish_openai(reason: str) -> str:
    return {"stop": "stop", "stop_sequence": "stop", "length": "length", "tool_calls": "tool_calls"}.get(reason, "stop")


def openai_chat_response(res: GenResult, model: str) -> dict:
    msg: Dict[str, object] = {"role": "assistant", "content": res.content or None}
    if res.reasoning:
        msg["reasoning_content"] = res.reasoning
    if res.tool_calls:
        msg["tool_calls"] = [{"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function",
                              "function": {"name": c.name, "arguments": c.arguments}} for c in res.tool_calls]
    return _with_boundary(
        {"id": f"chatcmpl-{res.request_id}", "object": "chat.completion", "created": int(time.time()), "model": model,
         "choices": [{"index": 0, "message": msg, "finish_reason": _finish_openai(res.finish_reason), "logprobs": None}],
         "usage": _usage_openai(res)}, res)


def openai_chat_stream(events: Iterator[tuple], model: str, include_usage: bool) -> Iterator[bytes]:
    cid, created = f"chatcmpl-{uuid.uuid4().hex[:24]}", int(time.time())

    def chunk(delta: dict, finish=None, usage=None, res=None) -> bytes:
        d = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model,
             "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
        if usage is not None:
            d["usage"] = usage
        return sse(_with_boundary(d, res) if res is not None else d)

    yield chunk({"role": "assistant", "content": ""})
    n_calls = 0
    for kind, item in events:
        if kind == "delta":
            d: ParsedDelta = item
            if d.reasoning:
                yield chunk({"reasoning_content": d.reasoning})
            if d.content:
                yield chunk({"content": d.content})
            for c in d.tool_calls:
                yield chunk({"tool_calls": [{"index": n_calls, "id": f"call_{uuid.uuid4().hex[:24]}", "type": "function",
                                             "function": {"name": c.name, "arguments": c.arguments}}]})
                n_calls += 1
        else:
            res: GenResult = item
            yield chunk({}, finish=_finish_openai(res.finish_reason), res=res)
            if include_usage:
                d = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model, "choices": [],
                     "usage": _usage_openai(res)}
                yield sse(d)
    yield sse("[DONE]")


# =========================================================================================================
# OpenAI responses
# =========================================================================================================
def responses_input_to_messages(body: dict, store: Optional[dict] = None) -> List[dict]:
    msgs: List[dict] = []
    prev = body.get("previous_response_id")
    if prev:
        if store is None or prev not in store:
            raise BadRequest(f"previous_response_id '{prev}' not found", "previous_response_id", "not_found")
        msgs.extend(store[prev]["_messages"])
    if body.get("instructions"):
        msgs.insert(0, {"role": "system", "content": body["instructions"]})
    inp = body.get("input")
    if isinstance(inp, str):
        msgs.append({"role": "user", "content": inp})
    elif isinstance(inp, list):
        for item in inp:
            t = item.get("type", "message")
            if t == "message":
                msgs.append({"role": item.get("role", "user"), "content": item.get("content")})
            elif t == "function_call":
                msgs.append({"role": "assistant", "content": "", "tool_calls": [
                    {"function": {"name": item.get("name"), "arguments": item.get("arguments", "{}")}}]})
            elif t == "function_call_output":
                msgs.append({"role": "tool", "content": item.get("output", "")})
            elif t == "reasoning":
                continue
            else:
                raise BadRequest(f"unsupported input item type '{t}'", "input")
    else:
        raise BadRequest("input must be a string or a list of items", "input")
    return msgs


def parse_openai_responses(body: dict, store: Optional[dict] = None) -> Tuple[GenRequest, dict]:
    msgs = responses_input_to_messages(body, store)
    tools = None
    if body.get("tools"):
        tools = []
        for t in body["tools"]:
            if t.get("type") != "function":
                raise BadRequest("only function tools are supported", "tools", "unsupported_parameter")
            tools.append({"type": "function", "function": {k: t.get(k) for k in ("name", "description", "parameters")}})
    reasoning = body.get("reasoning") or {}
    req = GenRequest(messages=msgs, tools=tools, max_tokens=int(body.get("max_output_tokens") or 512),
                     temperature=_num(body, "temperature", 0.0, 2.0), top_p=_num(body, "top_p", 0.0, 1.0),
                     enable_thinking=reasoning.get("effort", "medium") not in ("none", "minimal"),
                     soft_max_tokens=_soft_max(body, "soft_max_output_tokens", int(body.get("max_output_tokens") or 512)),
                     **_openai_cache_hints(body, msgs))
    return req, {"stream": bool(body.get("stream", False)), "store": bool(body.get("store", True)), "messages": msgs}


def openai_responses_object(res: GenResult, model: str, status: str = "completed") -> dict:
    out: List[dict] = []
    if res.reasoning:
        out.append({"id": f"rs_{uuid.uuid4().hex[:24]}", "type": "reasoning",
                    "summary": [], "content": [{"type": "reasoning_text", "text": res.reasoning}]})
    if res.content or not res.tool_calls:
        out.append({"id": f"msg_{uuid.uuid4().hex[:24]}", "type": "message", "role": "assistant", "status": "completed",
                    "content": [{"type": "output_text", "text": res.content, "annotations": []}]})
    for c in res.tool_calls:
        out.append({"id": f"fc_{uuid.uuid4().hex[:24]}", "type": "function_call", "status": "completed",
                    "call_id": f"call_{uuid.uuid4().hex[:24]}", "name": c.name, "arguments": c.arguments})
    incomplete = {"reason": "max_output_tokens"} if res.finish_reason == "length" else None
    return _with_boundary(
        {"id": f"resp_{res.request_id}", "object": "response", "created_at": int(time.time()),
         "status": "incomplete" if incomplete else status, "incomplete_details": incomplete, "model": model,
         "output": out, "output_text": res.content,
         "usage": {"input_tokens": res.prompt_tokens, "output_tokens": res.completion_tokens,
                   "total_tokens": res.prompt_tokens + res.completion_tokens,
                   "input_tokens_details": {"cached_tokens": int(getattr(res, "cached_tokens", 0) or 0)}}}, res)


def openai_responses_stream(events: Iterator[tuple], model: str, on_done=None) -> Iterator[bytes]:
    rid = f"resp_{uuid.uuid4().hex[:24]}"
    seq = 0

    def ev(name: str, payload: dict) -> bytes:
        nonlocal seq
        payload = {"type": name, "sequence_number": seq, **payload}
        seq += 1
        return sse(payload, name)

    base = {"id": rid, "object": "response", "created_at": int(time.time()), "status": "in_progress", "model": model,
            "output": []}
    yield ev("response.created", {"response": base})
    yield ev("response.in_progress", {"response": base})
    item_id = f"msg_{uuid.uuid4().hex[:24]}"
    opened = False
    for kind, item in events:
        if kind == "delta":
            d: ParsedDelta = item
            if d.reasoning:
                yield ev("response.reasoning_text.delta", {"item_id": "rs_0", "output_index": 0, "content_index": 0, "delta": d.reasoning})
            if d.content:
                if not opened:
                    opened = True
                    yield ev("response.output_item.added", {"output_index": 0, "item": {
                        "id": item_id, "type": "message", "role": "assistant", "status": "in_progress", "content": []}})
                    yield ev("response.content_part.added", {"item_id": item_id, "output_index": 0, "content_index": 0,
                                                             "part": {"type": "output_text", "text": "", "annotations": []}})
                yield ev("response.output_text.delta", {"item_id": item_id, "output_index": 0, "content_index": 0, "delta": d.content})
        else:
            res: GenResult = item
            obj = openai_responses_object(res, model)
            obj["id"] = rid
            if opened:
                yield ev("response.output_text.done", {"item_id": item_id, "output_index": 0, "content_index": 0, "text": res.content})
            if on_done is not None:
                on_done(obj, res)
            yield ev("response.completed" if obj["status"] == "completed" else "response.incomplete", {"response": obj})


# =========================================================================================================
# Anthropic messages
# =========================================================================================================
def _anthropic_blocks_to_messages(role: str, content) -> List[dict]:
    if isinstance(content, str):
        return [{"role": role, "content": content}]
    out: List[dict] = []
    text, calls = [], []
    for b in content or []:
        t = b.get("type")
        if t == "text":
            text.append(b.get("text", ""))
        elif t == "thinking":
            continue  # earlier reasoning is not replayed
        elif t == "tool_use":
            calls.append({"function": {"name": b.get("name"), "arguments": b.get("input", {})}})
        elif t == "tool_result":
            c = b.get("content", "")
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if p.get("type") == "text")
            out.append({"role": "tool", "content": c})
        elif t in ("image", "document"):
            text.append("<|vision_start|><|image_pad|><|vision_end|>")
        else:
            raise BadRequest(f"unsupported content block '{t}'", "messages")
    if text or calls:
        m: Dict[str, object] = {"role": role, "content": "".join(text)}
        if calls:
            m["tool_calls"] = calls
        out.insert(0, m)
    return out


def parse_anthropic_messages(body: dict) -> Tuple[GenRequest, dict]:
    if "max_tokens" not in body:
        raise BadRequest("max_tokens is required", "max_tokens")
    msgs: List[dict] = []
    breakpoints: List[int] = []
    system = body.get("system")
    if system:
        if isinstance(system, list):
            if any(_anthropic_cache_marked(b) for b in system):
                breakpoints.append(0)
            system = "".join(b.get("text", "") for b in system)
        msgs.append({"role": "system", "content": system})
    raw = body.get("messages")
    if not isinstance(raw, list) or not raw:
        raise BadRequest("messages must be a non-empty list", "messages")
    for m in raw:
        if m.get("role") not in ("user", "assistant"):
            raise BadRequest("message role must be user or assistant", "messages")
        msgs.extend(_anthropic_blocks_to_messages(m["role"], m.get("content")))
        blocks = m.get("content") if isinstance(m.get("content"), list) else []
        if any(_anthropic_cache_marked(b) for b in blocks):
            breakpoints.append(len(msgs) - 1)     # the boundary sits after the last message this turn produced
    tools = None
    if body.get("tools"):
        tools = [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                   "parameters": t.get("input_schema", {})}} for t in body["tools"]]
    th = body.get("thinking") or {}
    thinking = th.get("type") == "enabled"
    budget = th.get("budget_tokens") if thinking else None
    if budget is not None and (not isinstance(budget, int) or isinstance(budget, bool) or budget < 1):
        raise BadRequest("thinking.budget_tokens must be a positive integer", "thinking")
    req = GenRequest(messages=msgs, tools=tools, max_tokens=int(body["max_tokens"]), thinking_budget=budget,
                     temperature=_num(body, "temperature", 0.0, 1.0), top_p=_num(body, "top_p", 0.0, 1.0),
                     top_k=_num(body, "top_k", 1, 20, int), stop=_stops(body.get("stop_sequences")),
                     enable_thinking=thinking, cache_breakpoints=breakpoints,
                     soft_max_tokens=_soft_max(body, "soft_max_tokens", int(body["max_tokens"])))
    return req, {"stream": bool(body.get("stream", False))}


def _stop_reason_anthropic(reason: str) -> str:
    return {"stop": "end_turn", "length": "max_tokens", "stop_sequence": "stop_sequence",
            "tool_calls": "tool_use"}.get(reason, "end_turn")


def _thinking_signature(text: str) -> str:
    import hashlib
    return hashlib.sha256(("ninfer-fusion-b200:thinking:" + text).encode("utf-8")).hexdigest()


def anthropic_message_response(res: GenResult, model: str) -> dict:
    content: List[dict] = []
    if res.reasoning:
        content.append({"type": "thinking", "thinking": res.reasoning, "signature": _thinking_signature(res.reasoning)})
    if res.content or not res.tool_calls:
        content.append({"type": "text", "text": res.content})
    for c in res.tool_calls:
        try:
            inp = json.loads(c.arguments)
        except json.JSONDecodeError:
            inp = {"_raw": c.arguments}
        content.append({"type": "tool_use", "id": f"toolu_{uuid.uuid4().hex[:24]}", "name": c.name, "input": inp})
    return _with_boundary(
        {"id": f"msg_{res.request_id}", "type": "message", "role": "assistant", "model": model, "content": content,
         "stop_reason": _stop_reason_anthropic(res.finish_reason), "stop_sequence": None,
         # Anthropic counts cached reads apart from the computed input
         "usage": {"input_tokens": res.prompt_tokens - int(getattr(res, "cached_tokens", 0) or 0),
                   "cache_read_input_tokens": int(getattr(res, "cached_tokens", 0) or 0),
                   "cache_creation_input_tokens": 0, "output_tokens": res.completion_tokens}}, res)


def anthropic_stream(events: Iterator[tuple], model: str, prompt_tokens_hint: int = 0) -> Iterator[bytes]:
    mid = f"msg_{uuid.uuid4().hex[:24]}"
    yield sse({"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "model": model,
                                                    "content": [], "stop_reason": None, "stop_sequence": None,
                                                    "usage": {"input_tokens": prompt_tokens_hint, "output_tokens": 0}}},
              "message_start")
    index, open_kind = -1, None
    thinking_text = ""

    def close():
        nonlocal open_kind
        out = []
        if open_kind == "thinking":
            out.append(sse({"type": "content_block_delta", "index": index,
                            "delta": {"type": "signature_delta", "signature": _thinking_signature(thinking_text)}},
                           "content_block_delta"))
        if open_kind is not None:
            out.append(sse({"type": "content_block_stop", "index": index}, "content_block_stop"))
        open_kind = None
        return out

    def open_block(kind: str, block: dict):
        nonlocal index, open_kind
        out = close()
        index += 1
        open_kind = kind
        out.append(sse({"type": "content_block_start", "index": index, "content_block": block}, "content_block_start"))
        return out

    for kind, item in events:
        if kind == "delta":
            d: ParsedDelta = item
            if d.reasoning:
                if open_kind != "thinking":
                    yield from open_block("thinking", {"type": "thinking", "thinking": ""})
                thinking_text += d.reasoning
                yield sse({"type": "content_block_delta", "index": index, "delta": {"type": "thinking_delta", "thinking": d.reasoning}},
                          "content_block_delta")
            if d.content:
                if open_kind != "text":
                    yield from open_block("text", {"type": "text", "text": ""})
                yield sse({"type": "content_block_delta", "index": index, "delta": {"type": "text_delta", "text": d.content}},
                          "content_block_delta")
            for c in d.tool_calls:
                yield from open_block("tool_use", {"type": "tool_use", "id": f"toolu_{uuid.uuid4().hex[:24]}", "name": c.name, "input": {}})
                yield sse({"type": "content_block_delta", "index": index, "delta": {"type": "input_json_delta", "partial_json": c.arguments}},
                          "content_block_delta")
        else:
            res: GenResult = item
            yield from close()
            yield sse(_with_boundary({"type": "message_delta",
                                      "delta": {"stop_reason": _stop_reason_anthropic(res.finish_reason), "stop_sequence": None},
                                      "usage": {"input_tokens": res.prompt_tokens, "output_tokens": res.completion_tokens}}, res),
                      "message_delta")
            yield sse({"type": "message_stop"}, "message_stop")
