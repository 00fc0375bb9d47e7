"""Generation service: owns the engine, the tokenizer and the chat frontend; protocol gateways talk to it.

Counterpart of the reference's src/serve/generation_service.cpp (engine ownership, warm-up, request
admission) plus the family frontend session (prompt preparation, stop handling, output parsing).
"""
from __future__ import annotations

import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional, Sequence

from ..frontend.chat import OutputParser, ParsedDelta, ToolCall, render_chat, render_chat_spans
from ..frontend.tokenizer import StreamDecoder, Tokenizer
from ..runtime.engine import Engine, Event, RequestError, RequestOptions, ResourceError
from ..runtime.program import SamplingParams

# Sampling defaults per mode (docs/serving.md:711-716 of the reference): thinking / non-thinking.
DEFAULT_SAMPLING = {
    True: dict(temperature=1.0, top_p=0.95, top_k=20, presence_penalty=0.0),
    False: dict(temperature=0.7, top_p=0.80, top_k=20, presence_penalty=1.5),
}


@dataclass
class GenRequest:
    messages: Optional[List[dict]] = None      # chat form
    prompt: Optional[str] = None               # raw text form
    prompt_ids: Optional[List[int]] = None     # pre-tokenised form
    tools: Optional[List[dict]] = None
    max_tokens: int = 512
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    presence_penalty: Optional[float] = None
    frequency_penalty: Optional[float] = None
    seed: Optional[int] = None
    stop: Sequence[str] = ()
    enable_thinking: bool = True
    queue_timeout_s: Optional[float] = None
    deadline_s: Optional[float] = None
    session: Optional[str] = None
    thinking_budget: Optional[int] = None      # reasoning tokens after which the engine closes the reasoning frame
    # prompt-cache hints (OpenAI prompt_cache_options / prompt_cache_breakpoint, Anthropic cache_control): whether the
    # automatic shared-prefix candidate is written, and the messages after which the client asked for a boundary
    cache_implicit: bool = True
    cache_breakpoints: Sequence[int] = ()      # indices into `messages`; a boundary sits after that message
    cache_key: Optional[str] = None            # accepted client hint; not a session key, not a prefix identity
    cache_retention: Optional[str] = None      # accepted; residency follows the engine's retention classes
    # soft length limit: from this many completion tokens on, the generation ends at the next syntax-safe boundary
    # (frontend/stop_boundary.py) instead of running into max_tokens in the middle of a statement
    soft_max_tokens: Optional[int] = None
    # rows of the input-embedding space at declared columns of `prompt_ids` (runtime/inject.py): a payload object
    # {"dtype", "scale", "columns", "data"}; only with pre-tokenised prompts, only on programs that accept it
    inject: Optional[dict] = None


MAX_CACHE_WRITES = 4     # distinct shared-prefix write candidates one request may carry


@dataclass
class GenResult:
    request_id: str
    content: str = ""
    reasoning: str = ""
    tool_calls: List[ToolCall] = field(default_factory=list)
    finish_reason: str = "stop"       # stop | length | tool_calls | stop_sequence | cancelled | error | timeout
    prompt_tokens: int = 0
    completion_tokens: int = 0
    ttft_ms: Optional[float] = None
    total_s: float = 0.0
    error: str = ""
    token_ids: List[int] = field(default_factory=list)   # every committed completion token, in order
    cached_tokens: int = 0        # prompt tokens served from a retained frontier
    reuse_kind: str = ""          # engine name of that frontier's kind ("" = none)
    queue_wait_s: float = 0.0     # submit -> lane
    prefill_chunks: int = 0
    decode_rounds: int = 0
    device_wait_s: float = 0.0            # time of this request's units spent blocked on the device
    host_exposed_s: float = 0.0           # the rest of those units' wall time
    decode_device_wait_s: float = 0.0
    decode_host_exposed_s: float = 0.0
    speculative: Optional[dict] = None    # draft-verify counters of this request (None: ordinary decode)
    thinking_budget: Optional[int] = None
    thinking_budget_applied: bool = False
    thinking_tokens: int = 0
    stop_boundary: Optional[dict] = None  # out-of-band notice of a soft length limit: where the stop was taken / deferred


class GenerationService:
    def __init__(self, engine: Engine, tokenizer: Tokenizer, model_id: str, max_concurrent: int = 64,
                 queue_timeout_s: float = 30.0, eos_tokens: Sequence[str] = ("<|im_end|>", "<|endoftext|>")):
        self.engine, self.tok, self.model_id = engine, tokenizer, model_id
        self.queue_timeout_s = queue_timeout_s
        self.eos_ids = [i for i in (tokenizer.token_id(t) for t in eos_tokens) if i is not None]
        self._permits = threading.Semaphore(max_concurrent)
        self.max_concurrent = max_concurrent
        self.started = time.time()
        self.media = None                 # frontend.media.MediaProcessor, created on the first media request
        self.media_pool = None            # runtime.worker_pool.HostWorkerPool for media decoding / resizing
        self.auto_shared_prefix = True    # publish the leading system block of chat prompts in the shared-prefix catalogue
        self.min_shared_prefix_tokens = 32
        self.allow_media_files = False    # local paths in media parts (CLI use); gateways leave this off
        # process-level settings of the server's option table
        self.sampling_overrides: Dict[str, float] = {}   # replace the registered sampler defaults; a request's own value still wins
        self.force_greedy = False         # exact arg-max for every request, whatever it asks for
        self.fixed_seed: Optional[int] = None   # seed of requests that give none (default: a fresh one per request)
        self.prefix_reuse = True          # off: no session continuations, no shared prefixes, no replay frontiers
        self.media_threads = 4
        self.default_thinking_budget: Optional[int] = None   # inherited by thinking-enabled requests that name none
        # the reasoning frame in token ids (None when the tokenizer has no such tokens: budgets are then ignored)
        self._think_ids = (tokenizer.token_id("<think>"), tokenizer.token_id("</think>"))

    # ------------------------------------------------------------------ prompt side
    def prepare(self, req: GenRequest) -> List[int]:
        return self.prepare_full(req)[0]

    def prepare_full(self, req: GenRequest):
        """(token ids, prepared media prompt or None).  Image / video parts of chat messages go through the media
        processor: placeholders expand to one pad token per visual token and positions become three-axis."""
        if req.inject is not None:
            if req.prompt_ids is None:
                raise RequestError("injected rows address token columns: they need prompt_ids")
            from ..runtime.inject import InjectRefused, parse_injection
            try:
                return list(req.prompt_ids), parse_injection(req.inject, req.prompt_ids, self.engine.program.cfg.hidden)
            except InjectRefused as e:
                raise RequestError(f"invalid injection: {e}")
        if req.prompt_ids is not None:
            return list(req.prompt_ids), None
        if req.messages is not None:
            text, spans = render_chat_spans(req.messages, req.tools, add_generation_prompt=True,
                                            enable_thinking=req.enable_thinking)
            from ..frontend import media as M
            if M.collect_media(req.messages):
                if self.tok.spells_control(text, spans):
                    # the media path tokenises the expanded text as a whole: a message that spells a control token
                    # (a pad, an end-of-turn marker) would be read as one
                    raise RequestError("message text of a media prompt may not spell control tokens")
                if not getattr(self.engine.program, "supports_media", False):
                    raise RequestError("this deployment has no vision tower: image and video parts are not supported")
                if self.media is None:
                    self.media = M.MediaProcessor()
                try:
                    if self.media_pool is None:
                        from ..runtime.worker_pool import HostWorkerPool
                        self.media_pool = HostWorkerPool(threads=self.media_threads, queue_capacity=16)
                    pm = M.prepare_messages(self.tok, text, req.messages, self.media, allow_files=self.allow_media_files,
                                            pool=self.media_pool)
                except (ValueError, OSError) as e:
                    raise RequestError(f"invalid media: {e}")
                return list(pm.ids), pm
            # what the caller wrote is literal text: only the template's own fragments may become control tokens
            return self.tok.encode_framed(text, spans)[0], None
        elif req.prompt is not None:
            text = req.prompt     # a raw prompt is the caller's own template: control tokens are read as such
        else:
            raise RequestError("request has neither messages nor prompt")
        return self.tok.encode(text), None

    def prompt_origin(self, req: GenRequest) -> Tuple[List[int], List[int]]:
        """(token ids, origin per token) of a text-only chat request: 0 = the template wrote the token, 1 = it lies in
        the caller's literal text, 2 = it straddles an edge."""
        if req.messages is None:
            raise RequestError("only chat requests have a template / literal origin")
        text, spans = render_chat_spans(req.messages, req.tools, add_generation_prompt=True,
                                        enable_thinking=req.enable_thinking)
        return self.tok.encode_framed(text, spans)

    def _encode_chat(self, messages, tools, add_generation_prompt: bool, enable_thinking: bool,
                     until_first_frame_end: bool = False) -> List[int]:
        """Token ids of a rendered history under the same rule as `prepare_full` (literal text yields no control
        tokens); optionally only up to and including the first end-of-turn marker the TEMPLATE wrote."""
        text, spans = render_chat_spans(messages, tools, add_generation_prompt=add_generation_prompt,
                                        enable_thinking=enable_thinking)
        if until_first_frame_end:
            mark, at, end = "<|im_end|>\n", 0, -1
            while True:
                at = text.find(mark, at)
                if at < 0:
                    break
                if not any(a < at + len(mark) and b > at for a, b in spans):
                    end = at + len(mark)
                    break
                at += 1
            if end < 0:
                return []
            text, spans = text[:end], [(a, min(b, end)) for a, b in spans if a < end]
        return self.tok.encode_framed(text, spans)[0]

    def shared_prefix_tokens(self, req: GenRequest, ids: Sequence[int]) -> int:
        """Length in tokens of the prompt's leading system block (system / developer message with the tool
        declarations the template renders into it), when it is long enough to be worth sharing across sessions."""
        if not self.auto_shared_prefix or req.messages is None or not req.messages:
            return 0
        if req.messages[0].get("role") not in ("system", "developer") and not req.tools:
            return 0
        head = self._encode_chat(req.messages, req.tools, True, req.enable_thinking, until_first_frame_end=True)
        n = len(head)
        if n < self.min_shared_prefix_tokens or n >= len(ids) or list(ids[:n]) != head:
            return 0
        return n

    def shared_prefix_edges(self, req: GenRequest, ids: Sequence[int]) -> List[int]:
        """Token frontiers this request may publish in the shared-prefix catalogue, ascending: the implicit candidate
        (the leading system block, unless the client switched implicit writes off) and the latest explicit
        breakpoints, at most MAX_CACHE_WRITES distinct ones.  A breakpoint whose rendered history is not an exact
        token prefix of the prompt is ignored: the hints never change the prompt."""
        edges = set()
        if req.cache_implicit:
            n = self.shared_prefix_tokens(req, ids)
            if n:
                edges.add(n)
        explicit: List[int] = []
        if req.messages:
            for i in sorted({int(b) for b in req.cache_breakpoints if 0 <= int(b) < len(req.messages)}):
                head = self._encode_chat(req.messages[: i + 1], req.tools, False, req.enable_thinking)
                n = len(head)
                if self.min_shared_prefix_tokens <= n < len(ids) and list(ids[:n]) == head:
                    explicit.append(n)
        room = MAX_CACHE_WRITES - len(edges)
        for n in explicit[::-1]:                      # the latest boundaries win the remaining slots
            if n in edges:
                continue
            if room <= 0:
                break
            edges.add(n)
            room -= 1
        return sorted(edges)

    def replay_edge_tokens(self, req: GenRequest, ids: Sequence[int]) -> int:
        """Tokens of the rendered history without the generation opener (what the template appends to make the model
        answer): the frontier a regenerated response restarts from.  0 when the prompt is not a chat or the opener
        is not a clean token suffix."""
        if req.messages is None or not req.messages or not req.session:
            return 0
        head = self._encode_chat(req.messages, req.tools, False, req.enable_thinking)
        n = len(head)
        if n == 0 or n >= len(ids) or list(ids[:n]) != head:
            return 0
        return n

    def count_tokens(self, req: GenRequest) -> int:
        return len(self.prepare(req))

    def _options(self, req: GenRequest) -> RequestOptions:
        d = dict(DEFAULT_SAMPLING[bool(req.enable_thinking)])
        d.update(self.sampling_overrides)
        if self.fixed_seed is not None:
            d["seed"] = self.fixed_seed
        for k in ("temperature", "top_p", "top_k", "min_p", "presence_penalty", "frequency_penalty", "seed"):
            v = getattr(req, k)
            if v is not None:
                d[k] = v
        if self.force_greedy:
            d.update(temperature=0.0, top_k=1)
        sp = SamplingParams(temperature=float(d.get("temperature", 0.0)), top_k=int(d.get("top_k", 20)),
                            top_p=float(d.get("top_p", 1.0)), min_p=float(d.get("min_p", 0.0)),
                            presence_penalty=float(d.get("presence_penalty", 0.0)),
                            frequency_penalty=float(d.get("frequency_penalty", 0.0)), seed=int(d.get("seed", 0)))
        opts = RequestOptions(max_tokens=max(1, int(req.max_tokens)), sampling=sp, stop_token_ids=tuple(self.eos_ids),
                              deadline_s=req.deadline_s,
                              pending_timeout_s=req.queue_timeout_s if req.queue_timeout_s is not None else self.queue_timeout_s,
                              session=req.session if self.prefix_reuse else None)
        budget = req.thinking_budget if req.thinking_budget is not None else self.default_thinking_budget
        open_id, close_id = self._think_ids
        if budget is not None and budget > 0 and req.enable_thinking and open_id is not None and close_id is not None:
            opts.thinking_budget = int(budget)
            opts.think_open_id, opts.think_close_id = int(open_id), int(close_id)
            opts.think_close_ids = tuple(self.tok.encode("\n</think>\n\n"))
        return opts

    # ------------------------------------------------------------------ generation
    def stream(self, req: GenRequest, on_start: Optional[Callable[[str, int], None]] = None,
               cancelled: Optional[Callable[[], bool]] = None) -> Iterator[tuple]:
        """Yields ("delta", ParsedDelta) items and finally ("done", GenResult)."""
        rid = uuid.uuid4().hex[:24]
        if not self._permits.acquire(blocking=False):
            raise ResourceError("server_overloaded: too many requests in flight")
        t0 = time.perf_counter()
        res = GenResult(rid)
        try:
            ids, media = self.prepare_full(req)
            res.prompt_tokens = len(ids)
            if on_start is not None:
                on_start(rid, len(ids))
            opts = self._options(req)
            opts.media = media
            if media is None and self.prefix_reuse:
                edges = self.shared_prefix_edges(req, ids)
                opts.shared_prefix_edges = tuple(edges)
                opts.shared_prefix_tokens = edges[0] if edges else 0
                opts.replay_edge_tokens = self.replay_edge_tokens(req, ids)
            handle = self.engine.submit(ids, opts)
            dec = StreamDecoder(self.tok, skip_special=True)
            # a chat prompt with thinking enabled continues inside an open reasoning frame only if the template
            # opened one; this template leaves the frame to the model, so parsing starts in content mode
            parser = OutputParser(thinking=False, stop=req.stop)
            eos = set(self.eos_ids)
            scanner = soft_stop = None
            if req.soft_max_tokens is not None:
                from ..frontend.stop_boundary import BoundaryScanner, pause_notice
                scanner = BoundaryScanner()
            while True:
                try:
                    ev: Event = handle.events.get(timeout=0.25)
                except Exception:
                    if cancelled is not None and cancelled():
                        handle.cancel()
                    continue
                if ev.kind == "token":
                    res.completion_tokens += 1
                    res.token_ids.append(int(ev.token))
                    if ev.token in eos or soft_stop is not None:
                        continue               # after a soft stop: tokens the engine committed before it saw the cancel
                    piece = dec.feed(ev.token)
                    if scanner is not None:
                        where = scanner.observe_token(piece or "")
                        if res.completion_tokens >= req.soft_max_tokens and where.safe:
                            soft_stop = pause_notice(where, "soft_max_tokens")
                            handle.cancel()
                            res.finish_reason = "length"
                    d = parser.feed(piece) if piece else ParsedDelta()
                    if d.content or d.reasoning or d.tool_calls:
                        yield ("delta", d)
                    if parser.stopped:
                        handle.cancel()
                        res.finish_reason = "stop_sequence"
                elif ev.kind in ("done", "error"):
                    tail = parser.feed(dec.flush())
                    end = parser.finish()
                    tail.content += end.content
                    tail.reasoning += end.reasoning
                    if tail.content or tail.reasoning or tail.tool_calls:
                        yield ("delta", tail)
                    if ev.kind == "error":
                        res.finish_reason, res.error = "error", ev.message
                    elif res.finish_reason != "stop_sequence" and soft_stop is None:
                        res.finish_reason = ev.finish_reason or "stop"
                    if scanner is not None:
                        # taken at a boundary, or (the hard limit came first) how far from one the output ends
                        res.stop_boundary = soft_stop or (pause_notice(scanner.decision(), "max_tokens")
                                                          if res.finish_reason == "length" else None)
                    break
            res.content, res.reasoning, res.tool_calls = parser.content, parser.reasoning, list(parser.tool_calls)
            if res.tool_calls and res.finish_reason == "stop":
                res.finish_reason = "tool_calls"
            res.ttft_ms = handle.ttft_ms
            res.total_s = time.perf_counter() - t0
            res.cached_tokens, res.reuse_kind = handle.cached_tokens, handle.reuse_kind
            res.queue_wait_s = (handle.t_admit - handle.t_submit) if handle.t_admit is not None else 0.0
            res.prefill_chunks, res.decode_rounds = handle.prefill_chunks, handle.decode_rounds
            res.device_wait_s, res.host_exposed_s = handle.device_wait_s, handle.host_exposed_s
            res.decode_device_wait_s, res.decode_host_exposed_s = handle.decode_device_wait_s, handle.decode_host_exposed_s
            res.speculative = handle.speculative
            res.thinking_budget = opts.thinking_budget
            res.thinking_budget_applied, res.thinking_tokens = handle.thinking_budget_applied, handle.thinking_tokens
            yield ("done", res)
        finally:
            self._permits.release()

    def generate(self, req: GenRequest) -> GenResult:
        last = None
        for kind, item in self.stream(req):
            if kind == "done":
                last = item
        return last

    def health(self) -> dict:
        h = self.engine.health()
        h.update({"model": self.model_id, "uptime_s": round(time.time() - self.started, 1),
                  "stats": self.engine.stats.as_dict()})
        return h
