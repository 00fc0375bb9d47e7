"""Bounded host worker pool: results in order, back-pressure on a full queue, checkpoint-driven abandonment."""
import threading
import time

import pytest

from ninfer_fusion_b200.runtime.worker_pool import HostWorkerPool


def test_results_and_exceptions_come_back_through_futures():
    pool = HostWorkerPool(threads=3, queue_capacity=4)
    try:
        assert pool.map([(lambda i=i: i * i) for i in range(20)]) == [i * i for i in range(20)]
        f = pool.submit(lambda: 1 / 0)
        with pytest.raises(ZeroDivisionError):
            f.result(timeout=5)
        s = pool.snapshot()
        assert s.threads == 3 and s.queued == 0
    finally:
        pool.shutdown()


def test_full_queue_blocks_and_a_checkpoint_can_give_up():
    pool = HostWorkerPool(threads=1, queue_capacity=1)
    gate = threading.Event()
    try:
        first = pool.submit(gate.wait)            # occupies the only thread
        time.sleep(0.05)
        second = pool.submit(lambda: "queued")    # fills the only queue slot
        assert pool.snapshot().active == 1 and pool.snapshot().queued == 1
        calls = []

        def checkpoint():
            calls.append(1)
            if len(calls) >= 3:
                raise TimeoutError("deadline passed while waiting for a worker slot")

        with pytest.raises(TimeoutError):
            pool.submit(lambda: "never queued", checkpoint, poll_s=0.01)
        assert len(calls) == 3
        gate.set()
        assert first.result(timeout=5) is True and second.result(timeout=5) == "queued"
    finally:
        gate.set()
        pool.shutdown()
