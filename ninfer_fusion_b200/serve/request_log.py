"""JSONL request log of the gateway: one self-describing line per event.

Events and field names follow the reference's measurement log so that its consumers can read ours
(docs/serving.md:727-819 and :864-866 of the reference: schema name `ninfer_serve_request_log`, version 18):
`server_start | request_start | request_rejected | request_done | request_error | throughput`, every line with
`timestamp_unix_ms` and a process-unique `server_instance_id`; `request_done` carries the finish reason, prompt /
completion / cached / computed-prefill token counts, the prefix reuse path (`root | private_endpoint |
private_turn_closure | private_response_replay | private_long_anchor | shared_stable_prefix`), unrounded
`timings_seconds` (`prepare, ttft, vision, prefill, decode, total`), `engine_timing` (`queue_wait_seconds`, unit
counts, decode rounds) and a `speculative` object (`backend, draft_window, rounds, drafted_tokens, accepted_tokens,
fallback_steps, accepted_per_position`); `throughput` carries interval deltas and the scheduler gauges.  No response
text and no key material is ever written.  Fields the engine does not measure are present with null (the
reference's host-exposure phase split, its materialisation search diagnostics).
"""
from __future__ import annotations

import json
import os
import threading
import time
import uuid
from typing import Dict, Optional

SCHEMA_NAME = "ninfer_serve_request_log"
SCHEMA_VERSION = 18
EVENTS = ("server_start", "request_start", "request_rejected", "request_done", "request_error", "throughput")

# engine frontier kind -> the reference's reuse path names
REUSE_PATHS = {"": "root", "endpoint": "private_endpoint", "turn": "private_turn_closure", "replay": "private_response_replay",
               "anchor": "private_long_anchor", "shared": "shared_stable_prefix"}


def reuse_path(kind: str) -> str:
    return REUSE_PATHS.get(kind or "", "root")


def redact_argv(argv) -> list:
    """argv with the value of every key-like option replaced."""
    out, hide = [], False
    for a in argv:
        if hide:
            out.append("<redacted>")
            hide = False
            continue
        if a.startswith("--api-key="):
            out.append("--api-key=<redacted>")
            continue
        out.append(a)
        hide = a == "--api-key"
    return out


class RequestLog:
    def __init__(self, path: Optional[str] = None, throughput_every_s: float = 5.0):
        self._f = open(path, "a", buffering=1, encoding="utf-8") if path else None
        self._lock = threading.Lock()
        self._last_tp = time.time()
        self._every = throughput_every_s
        self._prev: Dict[str, float] = {}
        self.instance_id = f"{os.getpid():x}-{uuid.uuid4().hex[:12]}"
        self.lines = 0

    def event(self, kind: str, **fields) -> None:
        if kind not in EVENTS:
            raise ValueError(f"unknown log event '{kind}'")
        rec = {"schema": SCHEMA_NAME, "schema_version": SCHEMA_VERSION, "event": kind,
               "timestamp_unix_ms": int(time.time() * 1000), "server_instance_id": self.instance_id}
        rec.update(fields)
        with self._lock:
            self.lines += 1
            if self._f is not None:
                self._f.write(json.dumps(rec, ensure_ascii=False) + "\n")

    def request_done(self, res, api: str, stream: bool, speculative: Optional[dict] = None) -> None:
        """`res`: serve.service.GenResult of a finished (or failed) generation."""
        ttft = None if res.ttft_ms is None else res.ttft_ms / 1e3
        decode_s = None if ttft is None else max(0.0, res.total_s - ttft)
        fields = {
            "request_id": res.request_id, "protocol": api, "stream": bool(stream), "finish_reason": res.finish_reason,
            "tokens": {"prompt": res.prompt_tokens, "completion": res.completion_tokens, "cached": res.cached_tokens,
                       "computed_prefill": max(0, res.prompt_tokens - res.cached_tokens)},
            "reuse_path": reuse_path(res.reuse_kind),
            "timings_seconds": {"prepare": None, "ttft": ttft, "vision": None,
                                "prefill": None if ttft is None else max(0.0, ttft - res.queue_wait_s),
                                "decode": decode_s, "total": res.total_s},
            # host_exposed_seconds: the reference splits it into five phases (engine boundary, program submit / post,
            # commit, maintenance); this engine measures their sum per unit, so the phases are null and `total` is set
            "engine_timing": {"queue_wait_seconds": res.queue_wait_s,
                              "device_wait_exposed_seconds": getattr(res, "device_wait_s", None),
                              "host_exposed_seconds": {"engine_boundary": None, "program_submit": None, "program_post": None,
                                                       "engine_commit_output": None, "engine_maintenance": None,
                                                       "total": getattr(res, "host_exposed_s", None)},
                              "decode": {"rounds": res.decode_rounds,
                                         "host_exposed_seconds": getattr(res, "decode_host_exposed_s", None),
                                         "device_wait_seconds": getattr(res, "decode_device_wait_s", None)},
                              "units": {"prefill": res.prefill_chunks}},
            "speculative": speculative or {"backend": "none", "draft_window": 0, "rounds": 0, "drafted_tokens": 0,
                                           "accepted_tokens": 0, "fallback_steps": 0, "accepted_per_position": []},
            "materialization": None,
            "thinking_budget": {"budget": getattr(res, "thinking_budget", None),
                                "applied": bool(getattr(res, "thinking_budget_applied", False)),
                                "reasoning_tokens": int(getattr(res, "thinking_tokens", 0) or 0)},
            # soft length limit: where the stop was taken or how far from a boundary the hard limit cut (None: not asked)
            "stop_boundary": getattr(res, "stop_boundary", None),
        }
        if res.finish_reason == "error":
            fields["error"] = res.error
            self.event("request_error", **fields)
        else:
            self.event("request_done", **fields)

    def throughput(self, stats: dict, gauges: Optional[dict] = None) -> None:
        """Interval record (every `throughput_every_s`): counter deltas since the last record plus current gauges;
        fully idle intervals are omitted."""
        now = time.time()
        if now - self._last_tp < self._every:
            return
        dt = now - self._last_tp
        self._last_tp = now
        keys = ("prompt_tokens", "completion_tokens", "decode_rounds", "requests_done", "requests_failed",
                "requests_rejected", "prefix_hits", "prefix_tokens_reused", "host_prefill_s", "host_decode_s",
                "device_wait_prefill_s", "device_wait_decode_s")
        delta = {k: (stats.get(k, 0) or 0) - self._prev.get(k, 0) for k in keys}
        self._prev = {k: stats.get(k, 0) or 0 for k in keys}
        if not any(delta.values()):
            return
        rounds = delta["decode_rounds"]
        host_work = {"elapsed_seconds": {"total": delta["host_prefill_s"] + delta["host_decode_s"]},
                     "device_wait_seconds": delta["device_wait_prefill_s"] + delta["device_wait_decode_s"],
                     "work_class_seconds": {"decode": {"host": delta["host_decode_s"], "device_wait": delta["device_wait_decode_s"]},
                                            "prefill": {"host": delta["host_prefill_s"], "device_wait": delta["device_wait_prefill_s"]}},
                     "per_round": {"decode_host_us": (delta["host_decode_s"] / rounds * 1e6) if rounds else None,
                                   "decode_device_wait_us": (delta["device_wait_decode_s"] / rounds * 1e6) if rounds else None}}
        self.event("throughput", interval_seconds=dt,
                   prefill_tokens=delta["prompt_tokens"], decode_tokens=delta["completion_tokens"],
                   decode_rounds=rounds,
                   avg_decode_batch=(delta["completion_tokens"] / rounds) if rounds else None,
                   requests={"done": delta["requests_done"], "failed": delta["requests_failed"],
                             "rejected": delta["requests_rejected"]},
                   context_cache={"prefix_hits": delta["prefix_hits"], "prefix_tokens_reused": delta["prefix_tokens_reused"]},
                   host_work=host_work,
                   scheduler=gauges or {})

    def close(self) -> None:
        with self._lock:
            if self._f is not None:
                self._f.close()
                self._f = None
