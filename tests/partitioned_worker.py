"""One rank of the partitioned multi-rank engine tests (CPU, gloo): `python partitioned_worker.py SCENARIO RANK WORLD PORT OUT`.

Rank 0 runs an `Engine` over `PartitionedLeader`, the others `partitioned_follower_loop`, all around the CPU oracle
program with a counter of forward passes.  Scenarios: "lockstep" (every verb runs one forward pass on every rank),
"free" (idle ranks skip), "open_fault" (the owner refuses one lane), "leave" (the last rank exits between two verbs).
Every rank writes a JSON report to OUT.<rank>.
"""
import datetime
import json
import os
import sys

import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ninfer_fusion_b200.models.config import TINY_DENSE  # noqa: E402
from ninfer_fusion_b200.models.weights import random_weights  # noqa: E402
from ninfer_fusion_b200.parallel.partitioned import PartitionedLeader, partitioned_follower_loop  # noqa: E402
from ninfer_fusion_b200.parallel.replicated import RankChannel  # noqa: E402
from ninfer_fusion_b200.runtime.engine import Engine, RequestError, RequestOptions, ResourceError  # noqa: E402
from ninfer_fusion_b200.runtime.program import ReferenceProgram  # noqa: E402

CFG = TINY_DENSE.shrink(2)
W = random_weights(CFG, "cpu", seed=11, std=0.05)
PROMPTS = [[5, 9, 2, 7, 11], [3, 4, 8, 1, 6, 12, 40, 2, 9], [77, 3, 5], [8, 8, 1, 30, 2, 2, 19], [4, 4, 4, 9], [60, 2]]
N_NEW = 6


class CountingProgram(ReferenceProgram):
    """Oracle program that counts its forward passes and the token bound it was given for each."""

    def __init__(self, *a, refuse_open=None, **k):
        super().__init__(*a, **k)
        self.forwards, self.bounds, self.refuse_open, self.opens = 0, [], refuse_open, 0
        self._bound = None

    def set_global_tokens(self, n):
        self._bound = n

    def open(self, *a, **k):
        self.opens += 1
        if self.refuse_open is not None and self.opens == self.refuse_open:
            raise RequestError("injected: this rank refuses the lane")
        return super().open(*a, **k)

    def prefill_step(self, lane, budget):
        self.forwards += 1
        self.bounds.append(self._bound)
        return super().prefill_step(lane, budget)

    def decode_round(self, lanes):
        self.forwards += 1
        self.bounds.append(self._bound)
        return super().decode_round(lanes)


def main():
    scenario, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    report = {"rank": rank, "scenario": scenario}
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8.0))
    ch = RankChannel(None, rank, world)
    lockstep = scenario != "free"
    kw = {"refuse_open": 2} if scenario == "open_fault" and rank == 1 else {}     # (its scratch lane is open number 1)
    inner = CountingProgram(CFG, W, max_lanes=3, max_context=256, **kw)
    if rank != 0:
        seen = {"decode": 0}

        def on_verb(msg):
            if msg["op"] == "decode":
                seen["decode"] += 1
            if scenario == "leave" and rank == world - 1 and seen["decode"] == 3:
                report["left_after_decode_rounds"] = 2
                json.dump(report, open(f"{out}.{rank}", "w"))
                os._exit(0)      # between two verbs: nothing of this rank is in flight
        try:
            worker = partitioned_follower_loop(inner, ch, lockstep, on_verb)
            report.update(loop="stopped", forwards=inner.forwards, filler=worker.filler_steps, bounds=inner.bounds,
                          lanes_left=len(worker.lanes), free_lanes=inner.free_lanes())
        except ResourceError:
            report["loop"] = "channel_failed"
        json.dump(report, open(f"{out}.{rank}", "w"))
        return
    prog = {}

    def factory():
        prog["p"] = PartitionedLeader(inner, ch, lanes_per_rank=3, lockstep=lockstep)
        return prog["p"]
    eng = Engine(factory, prefill_chunk=4)
    handles = [eng.submit(p, RequestOptions(max_tokens=N_NEW)) for p in PROMPTS]
    results = []
    for h in handles:
        try:
            h.wait(timeout=120)
        except TimeoutError:
            pass
        results.append({"tokens": h.tokens, "reason": h.finish_reason, "error": h.error})
    report["results"] = results
    report["health"] = eng.health()["status"]
    if report["health"] == "ok":
        report["ping"] = prog["p"].ping()
        report["census"] = prog["p"].census()["partitioned"]
        report["forwards"], report["bounds"] = inner.forwards, inner.bounds
        prog["p"].shutdown()
    eng.shutdown()
    json.dump(report, open(f"{out}.0", "w"))


if __name__ == "__main__":
    main()
