"""Load progress on a terminal: one bar that rewrites its line, silent when stderr is not a TTY (logs stay clean).

Reference: src/product/load_progress (TTY progress bars while an artifact is materialised).
"""
from __future__ import annotations

import sys
import time
from typing import Optional


class Progress:
    def __init__(self, total: int, label: str = "", stream=None, force: Optional[bool] = None, width: int = 32):
        self.total, self.label, self.width = max(1, int(total)), label, width
        self.stream = stream if stream is not None else sys.stderr
        self.on = bool(force) if force is not None else bool(getattr(self.stream, "isatty", lambda: False)())
        self.done = 0
        self.t0 = time.perf_counter()
        self._last = 0.0

    def advance(self, n: int, what: str = "") -> None:
        self.done = min(self.total, self.done + int(n))
        now = time.perf_counter()
        if not self.on or (now - self._last < 0.05 and self.done < self.total):
            return
        self._last = now
        frac = self.done / self.total
        bar = "#" * int(frac * self.width)
        rate = self.done / max(1e-9, now - self.t0) / (1 << 20)
        self.stream.write(f"\r{self.label} [{bar:<{self.width}}] {100 * frac:5.1f}%  {rate:7.1f} MiB/s  {what[:40]:<40}")
        self.stream.flush()

    def close(self) -> None:
        if self.on:
            self.stream.write("\n")
            self.stream.flush()
