"""One rank of the multi-rank engine tests (CPU, gloo): `python replicated_worker.py SCENARIO RANK WORLD PORT OUT`.

Rank 0 runs an `Engine` over `LeaderProgram`, the others `follower_loop`, all around the CPU oracle program.
Scenarios: "plain" (concurrent requests, tokens must equal a single-process run), "open_fault" (a follower
refuses one lane while it is being opened), "veto" (a follower says no to the first admissions),
"leave" (the last rank exits between two steps; the survivors regroup and serve again).
Every rank writes a JSON report to OUT.<rank>.
"""
import datetime
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ninfer_fusion_b200.models.config import TINY_DENSE  # noqa: E402
from ninfer_fusion_b200.models.weights import random_weights  # noqa: E402
from ninfer_fusion_b200.parallel.replicated import (OP_DECODE, LeaderProgram, RankChannel,  # noqa: E402
                                                    follower_loop)
from ninfer_fusion_b200.runtime.engine import Engine, RequestError, RequestOptions, ResourceError  # noqa: E402
from ninfer_fusion_b200.runtime.program import ReferenceProgram  # noqa: E402

CFG = TINY_DENSE.shrink(2)
W = random_weights(CFG, "cpu", seed=11, std=0.05)
PROMPTS = [[5, 9, 2, 7, 11], [3, 4, 8, 1, 6, 12, 40, 2, 9], [77, 3, 5], [8, 8, 1, 30, 2, 2, 19]]


class FaultyProgram(ReferenceProgram):
    """Oracle program with host-side faults: refuse the n-th open, veto the first admissions."""

    def __init__(self, *a, refuse_open=None, veto_first=0, **k):
        super().__init__(*a, **k)
        self.refuse_open, self.veto_left, self.opens = refuse_open, veto_first, 0

    def open(self, *a, **k):
        self.opens += 1
        if self.refuse_open is not None and self.opens == self.refuse_open:
            raise RequestError("injected: this rank refuses the lane")
        return super().open(*a, **k)

    def can_admit(self, n_prompt, max_new):
        if self.veto_left > 0:
            self.veto_left -= 1
            return False
        return super().can_admit(n_prompt, max_new)


def init(rank, world, port, timeout_s=8.0):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))
    return RankChannel(None, rank, world)


def main():
    scenario, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    report = {"rank": rank, "scenario": scenario}
    ch = init(rank, world, port)
    kw = {}
    if scenario == "open_fault" and rank == 1:
        kw["refuse_open"] = 2
    if scenario == "veto" and rank == world - 1:
        kw["veto_first"] = 3
    inner = FaultyProgram(CFG, W, max_lanes=3, max_context=256, **kw)

    if rank != 0:
        steps = {"n": 0}

        def on_step(op):
            if op == OP_DECODE:
                steps["n"] += 1
            if scenario == "leave" and rank == world - 1 and steps["n"] == 3:
                report["left_after_decode_rounds"] = 2
                json.dump(report, open(f"{out}.{rank}", "w"))
                os._exit(0)      # between two steps: nothing of this rank is in flight

        try:
            report["loop"] = follower_loop(inner, ch, on_step)
        except ResourceError as e:
            report["loop"] = "channel_failed"
            report["error"] = str(e)[:200]
            if scenario == "leave":
                # survivors regroup on a fresh rendezvous and serve again
                dist.destroy_process_group()
                ch = init(rank, world - 1, port + 1)
                inner = FaultyProgram(CFG, W, max_lanes=3, max_context=256)
                report["loop_after_regroup"] = follower_loop(inner, ch)
        report["lanes_left"] = len(inner.lanes)
        report["free_lanes"] = inner.free_lanes()
        json.dump(report, open(f"{out}.{rank}", "w"))
        return

    state = {"ch": ch}

    def factory():
        return LeaderProgram(FaultyProgram(CFG, W, max_lanes=3, max_context=256), state["ch"])

    eng = Engine(lambda: LeaderProgram(inner, ch), prefill_chunk=4)
    handles = [eng.submit(p, RequestOptions(max_tokens=6)) for p in PROMPTS]
    results = []
    for h in handles:
        try:
            results.append({"tokens": h.wait(timeout=120), "reason": h.finish_reason, "error": h.error})
        except Exception as e:  # noqa: BLE001
            results.append({"error": f"{type(e).__name__}: {e}"[:200], "reason": h.finish_reason})
    report["results"] = results
    report["health"] = eng.health()["status"]
    report["stats"] = dict(eng.program.replicated_stats) if eng.health()["status"] == "ok" else None
    if scenario == "leave":
        # the engine failed as a whole; regroup with the survivors, recover, serve again
        dist.destroy_process_group()
        state["ch"] = init(0, world - 1, port + 1)
        eng._factory = factory
        eng.recover()
        report["health_after_recover"] = eng.health()["status"]
        report["after_recover"] = eng.generate(PROMPTS[0], RequestOptions(max_tokens=6))
    if eng.health()["status"] == "ok":
        report["ping"] = eng.program.ping()
        eng.program.shutdown()
    eng.shutdown()
    json.dump(report, open(f"{out}.{rank}", "w"))


if __name__ == "__main__":
    main()
