"""Phase tracing: NVTX ranges with a fixed vocabulary, plus a host-side span log.

Off by default (an unset knob changes nothing).  ``NINFER_NVTX=1`` pushes NVTX ranges named ``<category>/<name>`` around
engine phases, program steps, model layers and graph capture / replay, which is what a timeline tool shows;
``NINFER_TRACE_LOG=<path>`` appends one JSON line per closed span (category, name, milliseconds of host time, an
optional payload such as token counts) for runs where no profiler is attached.

Reference: src/core/nvtx.h (NVTX3 domain with fixed Name / Category enums around engine phases, rounds, layers, graph
capture and launch) and the NINFER_*_TRACE environment knobs (docs/features/instrumentation.md).
"""
from __future__ import annotations

import json
import os
import threading
import time
from contextlib import contextmanager
from typing import Optional

CATEGORIES = ("engine", "program", "model", "graph", "comm", "io")
NAMES = {
    "engine": ("admit", "prefill_chunk", "decode_round", "commit", "recover", "reload_kv"),
    "program": ("prefill_step", "decode_round", "verify_round", "draft", "checkpoint", "demote", "promote"),
    "model": ("embed", "attn_layer", "gdn_layer", "mlp", "moe", "logits", "vision_tower"),
    "graph": ("capture", "replay"),
    "comm": ("tp_reduce", "ep_dispatch", "ep_combine", "pp_handoff"),
    "io": ("artifact_load", "cold_write", "cold_read"),
}

_nvtx_on = os.environ.get("NINFER_NVTX") == "1"
_log_path = os.environ.get("NINFER_TRACE_LOG") or None
_lock = threading.Lock()


def configure(nvtx: Optional[bool] = None, log_path: Optional[str] = None) -> None:
    """Programmatic switch (tests, notebooks); None leaves a setting as it is, '' turns the log off."""
    global _nvtx_on, _log_path
    if nvtx is not None:
        _nvtx_on = bool(nvtx)
    if log_path is not None:
        _log_path = log_path or None


def enabled() -> bool:
    return _nvtx_on or _log_path is not None


def _nvtx():
    try:
        import torch
        return torch.cuda.nvtx if torch.cuda.is_available() else None
    except Exception:   # no torch / no CUDA runtime: ranges are skipped, the span log still works
        return None


@contextmanager
def span(category: str, name: str, **payload):
    """``with span("engine", "decode_round", lanes=8): ...``.  Names outside the vocabulary are refused so that a
    timeline never fills up with ad-hoc strings."""
    if not enabled():
        yield
        return
    if category not in NAMES or name not in NAMES[category]:
        raise ValueError(f"trace span {category}/{name} is not in the vocabulary")
    nv = _nvtx() if _nvtx_on else None
    if nv is not None:
        nv.range_push(f"{category}/{name}")
    t0 = time.perf_counter()
    try:
        yield
    finally:
        dt = (time.perf_counter() - t0) * 1e3
        if nv is not None:
            nv.range_pop()
        if _log_path is not None:
            rec = {"cat": category, "name": name, "ms": round(dt, 4), "t": round(time.time(), 6)}
            rec.update(payload)
            with _lock, open(_log_path, "a", encoding="utf-8") as f:
                f.write(json.dumps(rec) + "\n")
