"""JSONL request log of the gateway: one self-describing line per event.

Events: server_start | request_start | request_rejected | request_done | request_error | throughput
(docs/serving.md:737-750 of the reference; its schema carries a version so that consumers can refuse what
they do not understand).
"""
from __future__ import annotations

import json
import threading
import time
from typing import Optional

SCHEMA_VERSION = 1
EVENTS = ("server_start", "request_start", "request_rejected", "request_done", "request_error", "throughput")


class RequestLog:
    def __init__(self, path: Optional[str] = None, throughput_every_s: float = 10.0):
        self._f = open(path, "a", buffering=1, encoding="utf-8") if path else None
        self._lock = threading.Lock()
        self._last_tp = 0.0
        self._every = throughput_every_s
        self.lines = 0

    def event(self, kind: str, **fields) -> None:
        if kind not in EVENTS:
            raise ValueError(f"unknown log event '{kind}'")
        rec = {"schema": SCHEMA_VERSION, "ts": round(time.time(), 3), "event": kind}
        rec.update({k: v for k, v in fields.items() if v is not None})
        with self._lock:
            self.lines += 1
            if self._f is not None:
                self._f.write(json.dumps(rec, ensure_ascii=False) + "\n")

    def throughput(self, stats: dict, _elapsed: float) -> None:
        now = time.time()
        if now - self._last_tp < self._every:
            return
        self._last_tp = now
        self.event("throughput", decode_tok_s=round(stats.get("decode_tok_s", 0.0), 2),
                   prefill_tok_s=round(stats.get("prefill_tok_s", 0.0), 2), requests_done=stats.get("requests_done"),
                   requests_failed=stats.get("requests_failed"), completion_tokens=stats.get("completion_tokens"))

    def close(self) -> None:
        with self._lock:
            if self._f is not None:
                self._f.close()
                self._f = None
