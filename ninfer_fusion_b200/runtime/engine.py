"""Engine: the request control plane over a Program.

One worker thread owns every mutation (admission, prefill steps, decode rounds, commits); callers
submit requests and consume events from per-request queues.  Loop order per iteration: expire
deadlines -> settle cancellations -> admit FIFO heads while lanes / KV room allow -> advance ONE
prefill chunk (governed chunk size) -> one decode round over every decode-ready lane -> commit
(stop rules, budgets) -> publish.  Failures are classified Request / Resource / Invariant: a
request-domain failure fails only that lane, anything else poisons the engine until `recover()`
rebuilds the Program.  This keeps the reference's engine contract
(include/ninfer/engine.h:78-163, src/runtime/engine/engine_core.h: worker_loop :2248-2479,
commit ordering :1164, failure classification :454-496, lane failure :2148-2196, fault injection
:2118-2142, bandwidth governor src/runtime/engine/bandwidth_governor.h) with a batch envelope sized
for B200 (tens of lanes instead of 16).
"""
from __future__ import annotations

import os
import queue
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..utils import trace
from .program import Lane, ProgramBase, SamplingParams
from .scheduler import ExecutionAction, Scheduler, ServiceAccount, projected_service_work


class RequestError(Exception):
    """The request itself is at fault (bad arguments, too long, cancelled)."""


class ResourceError(Exception):
    """The engine ran out of something (lanes, KV pages, a device wait ran out)."""


class InvariantError(Exception):
    """Internal state is inconsistent; the engine must be rebuilt."""


@dataclass
class RequestOptions:
    max_tokens: int = 256
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_token_ids: Sequence[int] = ()
    deadline_s: Optional[float] = None       # wall-clock budget for the whole request
    pending_timeout_s: Optional[float] = None  # how long it may wait for admission
    session: Optional[str] = None            # continuation key for prefix reuse
    media: object = None                     # frontend.media.PreparedPrompt for a request with images / videos
    shared_prefix_tokens: int = 0            # publish the first N prompt tokens (system prompt) in the shared catalogue
    shared_prefix_edges: Sequence[int] = ()  # further token frontiers to publish there (explicit cache breakpoints)
    # thinking budget: after `thinking_budget` tokens inside an open reasoning frame the engine feeds `think_close_ids`
    # (the frame's closing sequence) instead of what the model sampled, then hands generation back to the model
    thinking_budget: Optional[int] = None
    think_open_id: int = -1
    think_close_id: int = -1
    think_close_ids: Sequence[int] = ()
    thinking_open_at_start: bool = False     # the prompt itself leaves a reasoning frame open
    replay_edge_tokens: int = 0              # session frontier before the generation opener (regenerate-this-response point)


@dataclass
class Event:
    kind: str                 # "token" | "done" | "error"
    token: int = -1
    finish_reason: str = ""   # "stop" | "length" | "cancelled" | "error" | "timeout"
    message: str = ""


@dataclass
class RuntimeStats:
    requests_submitted: int = 0
    requests_done: int = 0
    requests_failed: int = 0
    requests_rejected: int = 0
    prompt_tokens: int = 0
    completion_tokens: int = 0
    prefill_s: float = 0.0
    decode_s: float = 0.0
    decode_rounds: int = 0
    prefix_hits: int = 0
    prefix_tokens_reused: int = 0
    # the worker's wall time, each segment counted once whatever the batch size: host-active and device-wait seconds
    # per work class
    host_prefill_s: float = 0.0
    host_decode_s: float = 0.0
    device_wait_prefill_s: float = 0.0
    device_wait_decode_s: float = 0.0

    def as_dict(self) -> dict:
        d = dict(self.__dict__)
        d["decode_tok_s"] = self.completion_tokens / self.decode_s if self.decode_s > 0 else 0.0
        d["prefill_tok_s"] = self.prompt_tokens / self.prefill_s if self.prefill_s > 0 else 0.0
        return d


class GenerationHandle:
    def __init__(self, request_id: int):
        self.request_id = request_id
        self.events: "queue.Queue[Event]" = queue.Queue()
        self.tokens: List[int] = []
        self.finish_reason: str = ""
        self.error: str = ""
        self.t_submit = time.perf_counter()
        self.t_first: Optional[float] = None
        self.t_done: Optional[float] = None
        # filled by the worker: when the request got its lane, what it reused, how it was served
        self.t_admit: Optional[float] = None
        self.cached_tokens = 0          # prompt tokens restored from a retained frontier
        self.reuse_kind = ""            # kind of that frontier ("" = started at the root)
        self.prefill_chunks = 0
        self.decode_rounds = 0
        # wall time of the units this request took part in, split into time blocked on the device and host-active
        # time; in a batched round every participant is delayed by the whole round, so these explain one request's
        # latency and must not be summed across concurrent requests
        self.device_wait_s = 0.0
        self.host_exposed_s = 0.0
        self.decode_device_wait_s = 0.0
        self.decode_host_exposed_s = 0.0
        # draft-verify rounds this request took part in (a speculative program): what was drafted, what was accepted
        self.speculative: Optional[dict] = None
        self.thinking_budget_applied = False   # the engine closed this request's reasoning frame at its budget
        self.thinking_tokens = 0
        self._cancel = threading.Event()

    def cancel(self) -> None:
        self._cancel.set()

    @property
    def cancelled(self) -> bool:
        return self._cancel.is_set()

    def wait(self, sink: Optional[Callable[[Event], None]] = None, timeout: Optional[float] = None) -> List[int]:
        """Block until the request finishes; `sink` sees every event in publication order."""
        end = None if timeout is None else time.perf_counter() + timeout
        while True:
            left = None if end is None else max(0.0, end - time.perf_counter())
            try:
                ev = self.events.get(timeout=left)
            except queue.Empty:
                raise TimeoutError("generation did not finish in time") from None
            if sink is not None:
                sink(ev)
            if ev.kind in ("done", "error"):
                return self.tokens

    @property
    def ttft_ms(self) -> Optional[float]:
        return None if self.t_first is None else (self.t_first - self.t_submit) * 1e3


@dataclass
class _Request:
    handle: GenerationHandle
    prompt: List[int]
    opts: RequestOptions
    lane: Optional[Lane] = None
    state: str = "pending"     # pending | prefill | decode | finished
    n_generated: int = 0
    service: Optional[ServiceAccount] = None   # remaining work in quanta (prefill units + tokens to generate)
    borrower: bool = False                     # admitted past a blocked FIFO head
    thinking: bool = False                     # inside an open reasoning frame
    think_tokens: int = 0
    forced: Optional[list] = None              # control tokens still to be fed instead of sampled ones
    budget_applied: bool = False


def resolve_prefill_chunk_mode(cli_value: Optional[str] = None) -> str:
    """'dynamic' (the governor owns the prefill unit) or 'manual' (the unit stays what the caller asked for).
    Command line > environment (`NINFER_FT_BW_GOV`: 0 = manual, 1 = dynamic) > default (dynamic).  An unreadable value
    is refused by name rather than read as the default."""
    if cli_value:
        if cli_value not in ("dynamic", "manual"):
            raise ValueError(f"prefill chunk mode must be 'dynamic' or 'manual', got '{cli_value}'")
        return cli_value
    env = os.environ.get("NINFER_FT_BW_GOV")
    if env is None or env == "":
        return "dynamic"
    if env not in ("0", "1"):
        raise ValueError(f"NINFER_FT_BW_GOV must be 0 or 1, got '{env}'")
    return "dynamic" if env == "1" else "manual"


class BandwidthGovernor:
    """Paces prefill against decode: shrinks the prefill unit when decode rounds slow down, then thins the share of
    prefill units, and restores both when the rounds recover.

    Signal: the duration of a decode round against its own running floor (fastest recent rounds).  When a round that
    shared the loop with a prefill unit exceeds floor * tolerance the prefill unit halves (not below `min_unit`); once
    the unit is at its minimum the prefill SHARE halves instead (not below `min_share`): credit accrues `share` per
    completed decode round and a prefill unit costs one, so share 0.5 admits one prefill unit per two rounds and
    share 1 is the plain 1:1 alternation.  After `recover_rounds` clean rounds the share doubles back first, then the
    unit.  With no decode work the scheduler runs prefill whatever the credit (starvation is its business, not ours).
    `NINFER_FT_BW_TRACE=1` prints every change.  Reference: src/runtime/engine/bandwidth_governor.h."""

    def __init__(self, max_unit: int, min_unit: int = 128, tolerance: float = 1.5, recover_rounds: int = 8,
                 enabled: bool = True, min_share: float = 0.125):
        self.max_unit, self.min_unit = max_unit, min(min_unit, max_unit)
        self.unit = max_unit
        self.tolerance, self.recover_rounds = tolerance, recover_rounds
        self.enabled = enabled
        self.floor_ms: Optional[float] = None
        self._clean = 0
        self.share, self.min_share = 1.0, min_share
        self.credit = 1.0
        self._trace = os.environ.get("NINFER_FT_BW_TRACE", "") == "1"

    @property
    def mode(self) -> str:
        return "dynamic" if self.enabled else "manual"

    def _changed(self, why: str) -> None:
        if self._trace:
            print(f"[bandwidth governor] mode={self.mode} prefill unit={self.unit} share={self.share:g} ({why})",
                  file=sys.stderr, flush=True)

    # ---- consumption: asked at every decision point, charged when a prefill unit actually runs
    def prefill_allowed(self) -> bool:
        return not self.enabled or self.credit >= 1.0

    def charge_prefill(self) -> None:
        self.credit = max(0.0, self.credit - 1.0)

    def on_decode_round(self) -> None:
        self.credit = min(2.0, self.credit + self.share)

    def observe(self, decode_ms: float, shared_with_prefill: bool) -> None:
        if not self.enabled:
            return
        if not shared_with_prefill:
            self.floor_ms = decode_ms if self.floor_ms is None else min(self.floor_ms * 1.02, decode_ms) \
                if decode_ms < self.floor_ms * 1.02 else self.floor_ms
        if self.floor_ms is None:
            return
        if shared_with_prefill and decode_ms > self.floor_ms * self.tolerance:
            if self.unit > self.min_unit:
                self.unit = max(self.min_unit, self.unit // 2)
                self._changed("decode round above tolerance: unit halved")
            elif self.share > self.min_share:
                self.share = max(self.min_share, self.share / 2)
                self._changed("decode round above tolerance at the minimum unit: share halved")
            self._clean = 0
        else:
            self._clean += 1
            if self._clean >= self.recover_rounds:
                if self.share < 1.0:
                    self.share = min(1.0, self.share * 2)
                    self._clean = 0
                    self._changed("clean rounds: share doubled")
                elif self.unit < self.max_unit:
                    self.unit = min(self.max_unit, self.unit * 2)
                    self._clean = 0
                    self._changed("clean rounds: unit doubled")


class Engine:
    """Opaque engine facade: `submit()` from any thread, one worker thread does the rest."""

    def __init__(self, program_factory: Callable[[], ProgramBase], max_pending: int = 256,
                 prefill_chunk: int = 2048, governor: bool = True, prefill_chunk_mode: Optional[str] = None,
                 backfill_window: int = 8):
        self._factory = program_factory
        self.program = program_factory()
        # limits that submit() checks, cached so that it never touches the Program while the worker swaps it
        self._max_context = self.program.max_context
        self._supports_media = bool(getattr(self.program, "supports_media", False))
        self._reload = None      # (factory, done event, result box) posted by reload_kv_storage, served by the worker
        self.max_pending = max_pending
        # prefill unit: 'dynamic' = the governor owns it, 'manual' = it stays `prefill_chunk`
        mode = resolve_prefill_chunk_mode(prefill_chunk_mode) if governor else "manual"
        self.governor = BandwidthGovernor(prefill_chunk, enabled=mode == "dynamic")
        self.scheduler = Scheduler()
        self.backfill_window = backfill_window   # requests behind a blocked head that are looked at per iteration
        self._shared_round = False               # a prefill unit ran since the last decode round
        self.stats = RuntimeStats()
        self._pending: List[_Request] = []
        self._active: List[_Request] = []
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._next_id = 0
        self._failed: Optional[str] = None
        self._draining = False   # reload_kv_storage in progress: admission is paused
        self._stop = False
        self._fault = os.environ.get("NINFER_FAULT_INJECT", "")
        self._fault_min_id = int(os.environ.get("NINFER_FAULT_INJECT_MIN_ID", "0"))
        self._worker = threading.Thread(target=self._worker_loop, name="engine-worker", daemon=True)
        self._worker.start()

    # ------------------------------------------------------------------ public surface
    def submit(self, prompt: Sequence[int], opts: Optional[RequestOptions] = None) -> GenerationHandle:
        opts = opts or RequestOptions()
        with self._wake:
            if self._failed is not None:
                raise ResourceError(f"engine failed: {self._failed}; call recover()")
            if len(self._pending) >= self.max_pending:
                self.stats.requests_rejected += 1
                raise ResourceError("server_overloaded: pending queue is full")
            if len(prompt) == 0:
                raise RequestError("empty prompt")
            if opts.media is not None and getattr(opts.media, "items", None):
                if not self._supports_media:
                    raise RequestError("this engine has no vision tower: media prompts are not supported")
                if list(opts.media.ids) != list(prompt):
                    raise RequestError("the prepared media prompt does not match the request's token ids")
            elif opts.media is not None and getattr(opts.media, "rows", None) is not None:
                if not getattr(self.program, "supports_injection", False):
                    raise RequestError("this engine's program does not accept injected embedding rows")
                if list(opts.media.ids) != list(prompt):
                    raise RequestError("the injected prompt does not match the request's token ids")
            if len(prompt) + opts.max_tokens > self._max_context:
                self.stats.requests_rejected += 1
                raise RequestError(f"prompt ({len(prompt)}) + max_tokens ({opts.max_tokens}) exceeds the "
                                   f"context window ({self._max_context})")
            h = GenerationHandle(self._next_id)
            self._next_id += 1
            self._pending.append(_Request(h, list(prompt), opts))
            self.stats.requests_submitted += 1
            self._wake.notify_all()
            return h

    def generate(self, prompt: Sequence[int], opts: Optional[RequestOptions] = None) -> List[int]:
        return self.submit(prompt, opts).wait()

    def health(self) -> dict:
        with self._lock:
            prog = self.program   # None for the moment in which the worker rebuilds it (storage reload)
            out = {"status": "failed" if self._failed else "ok", "pending": len(self._pending),
                   "active": len(self._active), "free_lanes": prog.free_lanes() if prog is not None else 0}
            out["scheduler"] = dict(self.scheduler.stats, blocked_head=self.scheduler.protection is not None)
            out["prefill_pacing"] = {"mode": self.governor.mode, "unit": self.governor.unit, "share": self.governor.share}
        census = getattr(prog, "census", None)
        if census is not None:
            try:   # counts only (no tokens, no session names); the worker may be changing the catalogue meanwhile
                out["census"] = census()
            except Exception:
                pass
        return out

    def reload_kv_storage(self, program_factory: Callable[[], ProgramBase], timeout_s: float = 60.0) -> None:
        """Swap the KV storage plan (per-layer formats, page geometry) by rebuilding the Program once the engine has
        drained: new requests keep queueing, in-flight ones finish first.  Session checkpoints are dropped with the
        old Program.  (Reference: Engine::reload_kv_storage, src/runtime/engine/engine.cpp:764, used by the
        serve-side KV auto-relayout.)"""
        # The swap itself happens on the worker thread, the only thread that opens lanes: it serves the request
        # at the top of an iteration once no lane is active, so no admission can interleave with it, and it
        # builds the new Program outside the lock (submit() and health() keep answering meanwhile).
        done = threading.Event()
        box: dict = {}
        with self._wake:
            if self._reload is not None:
                raise ResourceError("a storage reload is already in progress")
            self._reload = (program_factory, done, box)
            self._draining = True
            self._wake.notify_all()
        if not done.wait(timeout_s):
            with self._wake:
                if self._reload is not None and not box.get("started"):
                    self._reload = None
                    self._draining = False
                    self._wake.notify_all()
                    raise TimeoutError("engine did not drain in time")
            done.wait()   # the worker is already building the new Program: let it finish
        if "error" in box:
            raise box["error"]

    def _serve_reload(self) -> None:
        """Worker thread, no lane active: replace the Program by the one the posted factory builds."""
        with self._lock:
            if self._reload is None:
                return
            factory, done, box = self._reload
            box["started"] = True
            old, self.program = self.program, None
        del old   # its device memory goes back before the new pools are allocated
        try:
            new = factory()
            with self._wake:
                self.program = new
                self._factory = factory
                self._max_context = new.max_context
                self._supports_media = bool(getattr(new, "supports_media", False))
        except Exception as e:  # noqa: BLE001 - the old Program is gone: engine-wide failure until recover()
            box["error"] = e
            with self._wake:
                self._failed = f"storage reload failed: {type(e).__name__}: {e}"
        finally:
            with self._wake:
                self._reload = None
                self._draining = False
                self._wake.notify_all()
            done.set()

    def recover(self) -> None:
        """Rebuild the Program after an engine-wide failure; in-flight requests were already failed."""
        with self._wake:
            if self._failed is None:
                return
            self.program = self._factory()
            self._max_context = self.program.max_context
            self._supports_media = bool(getattr(self.program, "supports_media", False))
            self._failed = None
            self._wake.notify_all()

    def shutdown(self) -> None:
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        self._worker.join(timeout=10)

    # ------------------------------------------------------------------ worker
    def _publish(self, req: _Request, ev: Event) -> None:
        h = req.handle
        if ev.kind == "token":
            if h.t_first is None:
                h.t_first = time.perf_counter()
            h.tokens.append(ev.token)
        else:
            h.finish_reason = ev.finish_reason
            h.error = ev.message
            h.t_done = time.perf_counter()
        h.events.put(ev)

    def _finish(self, req: _Request, reason: str, message: str = "") -> None:
        if req.state == "finished":
            return
        req.state = "finished"
        if req.lane is not None:
            if req.opts.session and reason in ("stop", "length"):
                self.program.checkpoint(req.lane, req.opts.session, "endpoint")   # where this turn's generation ended
            self.program.close(req.lane)
            req.lane = None
        if reason == "error":
            self.stats.requests_failed += 1
            self._publish(req, Event("error", finish_reason="error", message=message))
        else:
            self.stats.requests_done += 1
            self._publish(req, Event("done", finish_reason=reason))

    def _control(self, req: _Request, tok: int, last_of_round: bool) -> int:
        """Thinking budget.  Returns the token that is committed in place of the sampled `tok`: a pending control
        token when there is one and the sampled token has not been fed yet (it is the round's last), else `tok`."""
        o = req.opts
        if o.thinking_budget is None:
            return tok
        if req.n_generated == 0:
            req.thinking = bool(o.thinking_open_at_start)
        forced = bool(req.forced) and last_of_round
        if forced:
            tok = int(req.forced.pop(0))
            force = getattr(self.program, "force_next_token", None)
            if force is not None:
                force(req.lane, tok)          # the sampled token was only a proposal: this one is fed next
            else:
                req.lane.last_token = tok
        if tok == o.think_open_id:
            req.thinking = True
        elif tok == o.think_close_id:
            req.thinking = False
        elif req.thinking and not forced:
            req.think_tokens += 1
            req.handle.thinking_tokens = req.think_tokens
            if req.think_tokens >= o.thinking_budget and not req.budget_applied and o.think_close_ids:
                req.forced = [int(t) for t in o.think_close_ids]
                req.budget_applied = req.handle.thinking_budget_applied = True
        return tok

    def _commit_token(self, req: _Request, tok: int, last_of_round: bool = True) -> None:
        """Commit-before-publish: budget and stop rules are applied before the token becomes visible."""
        tok = self._control(req, tok, last_of_round)
        req.n_generated += 1
        self.stats.completion_tokens += 1
        if req.service is not None and req.service.remaining > 0:
            req.service.consume(1)
        if tok in req.opts.stop_token_ids:
            self._finish(req, "stop")
            return
        self._publish(req, Event("token", token=tok))
        if req.n_generated >= req.opts.max_tokens:
            self._finish(req, "length")

    def _maybe_inject(self, req: _Request) -> None:
        if self._fault and req.handle.request_id >= self._fault_min_id:
            kind, self._fault = self._fault, ""
            if kind == "request_once":
                raise RequestError("injected request fault")
            if kind == "invariant_once":
                raise InvariantError("injected invariant fault")

    def _open(self, req: _Request) -> None:
        """Gives `req` its lane (the caller has removed it from the pending queue)."""
        try:
            self._maybe_inject(req)
            req.lane = (self.program.open(req.prompt, req.opts.sampling, session=req.opts.session)
                        if req.opts.media is None else
                        self.program.open(req.prompt, req.opts.sampling, session=req.opts.session, media=req.opts.media))
            reserve = getattr(self.program, "reserve", None)
            if reserve is not None:
                # the pages this request may still grow into are spoken for from now on: a later admission
                # must not count them as free
                reserve(req.lane, len(req.prompt) + req.opts.max_tokens)
            req.handle.t_admit = time.perf_counter()
            if req.lane.reused:
                self.stats.prefix_hits += 1
                self.stats.prefix_tokens_reused += req.lane.reused
                req.handle.cached_tokens = int(req.lane.reused)
                req.handle.reuse_kind = getattr(req.lane, "reuse_kind", "") or "turn"
            left = len(req.prompt) - req.lane.n_cached
            req.service = ServiceAccount(projected_service_work(left, self.governor.unit, req.opts.max_tokens),
                                         self.governor.unit)
            req.state = "prefill"
            self._active.append(req)
        except RequestError as e:
            self._finish(req, "error", str(e))
        except Exception:
            self._active.append(req)  # it must be among the victims of the engine-wide failure
            raise

    def _admit(self) -> None:
        """FIFO admission.  A head that does not fit freezes the active requests as its donors; requests behind it
        are admitted out of order only with the Program's proof that the head still fits once the donors have left
        (runtime/scheduler.py)."""
        if self._draining or self.program is None:
            time.sleep(0.002)   # a storage reload is waiting for the lanes to drain
            return
        now = time.perf_counter()
        with self._lock:
            pend = list(self._pending)
        head: Optional[_Request] = None
        looked = 0
        for req in pend:
            if req.handle.cancelled:
                with self._lock:
                    self._pending.remove(req)
                self._finish(req, "cancelled")
                continue
            t_wait = req.opts.pending_timeout_s
            if t_wait is not None and now - req.handle.t_submit > t_wait:
                with self._lock:
                    self._pending.remove(req)
                self._finish(req, "error", "request_queue_timeout")
                continue
            if head is None:
                self.scheduler.observe_head(req.handle.request_id)
                if self.program.can_admit(len(req.prompt), req.opts.max_tokens):
                    with self._lock:
                        self._pending.remove(req)
                    self._open(req)
                    continue
                head = req
                self.scheduler.protect(req.handle.request_id, [r.handle.request_id for r in self._active])
                continue
            # behind a blocked head
            looked += 1
            if looked > self.backfill_window:
                break
            proof_fn = getattr(self.program, "admission_proof", None)
            if proof_fn is None or not self.program.can_admit(len(req.prompt), req.opts.max_tokens):
                continue
            prot = self.scheduler.protection
            active_ids = [r.handle.request_id for r in self._active]
            donors = [r.lane for r in self._active if r.handle.request_id in prot.donors and r.lane is not None]
            proof = proof_fn(len(head.prompt) + head.opts.max_tokens, len(req.prompt) + req.opts.max_tokens, donors)
            if self.scheduler.authorize_backfill(req.handle.request_id, active_ids, proof):
                with self._lock:
                    self._pending.remove(req)
                req.borrower = True
                self._open(req)
        if head is None:
            self.scheduler.observe_head(None)

    def _prefill_unit(self, req: _Request) -> None:
        """One prefill unit of `req` (at most the governor's unit, cut at a frontier boundary)."""
        t0 = time.perf_counter()
        w0 = getattr(self.program, "device_wait_s", 0.0)
        try:
            n_before = req.lane.n_cached
            budget = self.governor.unit
            if req.service is not None and req.service.unit != budget:
                req.service.reconcile(len(req.prompt) - n_before, budget)   # the unit moved under this request
            shared_edges = sorted({int(e) for e in (req.opts.shared_prefix_tokens, *req.opts.shared_prefix_edges) if e})
            replay = req.opts.replay_edge_tokens if req.opts.session else 0
            for e in (*shared_edges, replay):
                if 0 < e < len(req.prompt) and n_before < e:
                    budget = min(budget, e - n_before)     # stop exactly at the boundary
            with trace.span("engine", "prefill_chunk", budget=int(budget), cached=int(n_before)):
                first = self.program.prefill_step(req.lane, budget)
            req.handle.prefill_chunks += 1
            if req.service is not None and req.service.remaining > req.opts.max_tokens - req.n_generated:
                # one quantum per completed unit, out of the prefill part of the reservation only (a unit cut short
                # at a frontier boundary is one more unit than the projection counted)
                req.service.consume(1)
            self.stats.prompt_tokens += req.lane.n_cached - n_before
            if first is None and req.lane.n_cached in shared_edges and n_before < req.lane.n_cached:
                self.program.checkpoint(req.lane, "shared", "shared")   # any session may start from here
            if first is None and req.lane.n_cached == replay and n_before < replay:
                # the history up to, not including, the generation opener: a request that asks for this
                # response again (other sampling, other opener) starts here
                self.program.checkpoint(req.lane, req.opts.session, "replay")
            step = getattr(self.program, "anchor_interval", 0)
            if first is None and step > 0 and req.opts.session and req.lane.n_cached // step > n_before // step:
                self.program.checkpoint(req.lane, req.opts.session, "anchor")   # recovery point inside a long prompt
        except RequestError as e:
            self._active.remove(req)
            self._finish(req, "error", str(e))
            return
        dt = time.perf_counter() - t0
        wait = min(dt, max(0.0, getattr(self.program, "device_wait_s", 0.0) - w0))
        self.stats.prefill_s += dt
        self.stats.device_wait_prefill_s += wait
        self.stats.host_prefill_s += dt - wait
        req.handle.device_wait_s += wait
        req.handle.host_exposed_s += dt - wait
        if first is not None:
            if req.opts.session:
                self.program.checkpoint(req.lane, req.opts.session, "turn")   # the prompt boundary
            req.state = "decode"
            self._commit_token(req, first)

    def _decode_unit(self, ready: List[_Request]) -> None:
        """One decode round over the decode-ready lanes."""
        t0 = time.perf_counter()
        w0 = getattr(self.program, "device_wait_s", 0.0)
        with trace.span("engine", "decode_round", lanes=len(ready)):
            toks = self.program.decode_round([r.lane for r in ready])
        dt = time.perf_counter() - t0
        wait = min(dt, max(0.0, getattr(self.program, "device_wait_s", 0.0) - w0))
        self.stats.device_wait_decode_s += wait
        self.stats.host_decode_s += dt - wait
        for r in ready:
            r.handle.device_wait_s += wait
            r.handle.host_exposed_s += dt - wait
            r.handle.decode_device_wait_s += wait
            r.handle.decode_host_exposed_s += dt - wait
        self.stats.decode_s += dt
        self.stats.decode_rounds += 1
        self.governor.observe(dt * 1e3, self._shared_round)
        self.governor.on_decode_round()
        self._shared_round = False
        descend = getattr(self.program, "kv_descent_step", None)
        if descend is not None:
            descend()   # per-cell KV precision descent between rounds (a no-op unless the program is set up for it)
        for r in ready:
            r.handle.decode_rounds += 1
        for r, t in zip(ready, toks):
            if isinstance(t, (list, tuple)):
                window = int(getattr(self.program, "draft_window", 0) or max(0, len(t) - 1))
                sp = r.handle.speculative
                if sp is None:
                    sp = r.handle.speculative = {"backend": getattr(self.program, "speculative_backend", "mtp"),
                                                 "draft_window": window, "rounds": 0, "drafted_tokens": 0,
                                                 "accepted_tokens": 0, "fallback_steps": 0, "accepted_per_position": []}
                sp["rounds"] += 1
                sp["draft_window"] = max(sp["draft_window"], window)
                sp["drafted_tokens"] += window
                sp["accepted_tokens"] += len(t) - 1
                per = sp["accepted_per_position"]
                per.extend([0] * (len(t) - 1 - len(per)))
                for j in range(len(t) - 1):
                    per[j] += 1
            # a speculative program returns several tokens per lane and round; each one goes through the
            # same commit-before-publish gate, and nothing after a stop / budget hit becomes visible
            seq = t if isinstance(t, (list, tuple)) else (t,)
            for j, tok in enumerate(seq):
                if r.state == "finished":
                    break
                self._commit_token(r, tok, last_of_round=j == len(seq) - 1)

    def _worker_loop(self) -> None:
        while True:
            with self._wake:
                while not self._stop and (self._failed is not None or
                                          (not self._pending and not self._active and self._reload is None)):
                    self._wake.wait(timeout=0.5)
                if self._stop:
                    break
            try:
                self._iteration()
            except Exception as e:  # noqa: BLE001 - any escape from an iteration is an engine-wide failure, never a hang
                # engine-wide failure: fail every in-flight request, refuse new ones until recover()
                with self._lock:
                    self._failed = f"{type(e).__name__}: {e}"
                    victims = self._active + self._pending
                    self._active, self._pending = [], []
                for req in victims:
                    req.lane = None  # the Program is discarded as a whole
                    self._finish(req, "error", self._failed)

    def _iteration(self) -> None:
        if self._reload is not None and not self._active:
            self._serve_reload()
            if self._failed is not None:
                return
        now = time.perf_counter()
        for req in list(self._active):
            if req.handle.cancelled:
                self._active.remove(req)
                self._finish(req, "cancelled")
            elif req.opts.deadline_s is not None and now - req.handle.t_submit > req.opts.deadline_s:
                self._active.remove(req)
                self._finish(req, "timeout")
        self._admit()
        pre = next((r for r in self._active if r.state == "prefill"), None)
        ready = [r for r in self._active if r.state == "decode"]
        action = self.scheduler.choose(bool(ready), pre is not None, self.governor.prefill_allowed())
        if action is ExecutionAction.PREFILL:
            self._prefill_unit(pre)
            self.governor.charge_prefill()
            self._shared_round = True
        elif action is ExecutionAction.DECODE:
            self._decode_unit(ready)
        else:
            time.sleep(0.001)   # nothing runnable: a head that does not fit is waiting for its time-out or its donors
        self.scheduler.ran(action)
        self._active = [r for r in self._active if r.state != "finished"]
