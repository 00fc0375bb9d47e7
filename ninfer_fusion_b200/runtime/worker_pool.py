"""Bounded host worker pool for ordinary host work (media decoding and resizing, tokenising large prompts).

A fixed number of threads and a bounded FIFO: `submit` blocks while the queue is full (back-pressure instead of
unbounded memory) and, while it blocks, calls the caller's `checkpoint` so that a request that was cancelled or ran
past its deadline can give up instead of queueing.  The pool owns threads and the queue only; task semantics,
cancellation and result lifetime stay with the caller.  Counterpart of the reference's HostWorkerPool
(src/core/host_worker_pool.h: `submit(function, checkpoint) -> future`, `snapshot() -> {threads, queued, active}`).
"""
from __future__ import annotations

import queue
import threading
from concurrent.futures import Future
from dataclasses import dataclass
from typing import Callable, Optional


@dataclass(frozen=True)
class PoolSnapshot:
    threads: int
    queued: int
    active: int


class HostWorkerPool:
    def __init__(self, threads: int = 4, queue_capacity: int = 16):
        if threads < 1 or queue_capacity < 1:
            raise ValueError("a worker pool needs at least one thread and one queue slot")
        self._q: "queue.Queue" = queue.Queue(maxsize=queue_capacity)
        self._active = 0
        self._lock = threading.Lock()
        self._closed = False
        self._threads = [threading.Thread(target=self._run, name=f"host-worker-{i}", daemon=True) for i in range(threads)]
        for t in self._threads:
            t.start()

    def submit(self, fn: Callable[[], object], checkpoint: Optional[Callable[[], None]] = None,
               poll_s: float = 0.05) -> Future:
        """Queues `fn`; returns its future.  Blocks while the queue is full; `checkpoint()` runs between attempts and
        may raise to abandon the submission (nothing is queued then)."""
        if self._closed:
            raise RuntimeError("worker pool is shut down")
        fut: Future = Future()
        while True:
            try:
                self._q.put((fn, fut), timeout=poll_s)
                return fut
            except queue.Full:
                if checkpoint is not None:
                    checkpoint()

    def map(self, fns, checkpoint: Optional[Callable[[], None]] = None) -> list:
        """Runs the callables on the pool and returns their results in order (the first exception is re-raised)."""
        futs = [self.submit(f, checkpoint) for f in fns]
        return [f.result() for f in futs]

    def snapshot(self) -> PoolSnapshot:
        with self._lock:
            return PoolSnapshot(len(self._threads), self._q.qsize(), self._active)

    def shutdown(self) -> None:
        self._closed = True
        for _ in self._threads:
            self._q.put(None)
        for t in self._threads:
            t.join(timeout=5)

    def _run(self) -> None:
        while True:
            item = self._q.get()
            if item is None:
                return
            fn, fut = item
            if not fut.set_running_or_notify_cancel():
                continue
            with self._lock:
                self._active += 1
            try:
                fut.set_result(fn())
            except BaseException as e:  # noqa: BLE001 - the caller sees it through the future
                fut.set_exception(e)
            finally:
                with self._lock:
                    self._active -= 1
