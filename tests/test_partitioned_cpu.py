"""Partitioned multi-rank engine on CPU ranks (gloo): every request lives on one rank, one leader schedules them all,
lock step keeps the ranks' forward-pass counts equal, a refusing owner fails one request, a leaving rank fails the engine."""
import json
import os
import socket
import subprocess
import sys

import torch

from ninfer_fusion_b200.models.reference_model import ReferenceModel

WORKER = os.path.join(os.path.dirname(__file__), "partitioned_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(scenario, world, tmp_path):
    port = _free_port()
    out = str(tmp_path / "report")
    procs = [subprocess.Popen([sys.executable, WORKER, scenario, str(r), str(world), str(port), out],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    logs = []
    for p in procs:
        try:
            logs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            logs.append(p.communicate()[0] + "\nTIMEOUT")
    reports = []
    for r in range(world):
        path = f"{out}.{r}"
        assert os.path.exists(path), f"rank {r} wrote no report:\n{logs[r][-3000:]}"
        reports.append(json.load(open(path)))
    return reports


def _expected():
    from tests.partitioned_worker import CFG, N_NEW, PROMPTS, W
    ref = ReferenceModel(CFG, W)
    return [ref.generate_greedy(torch.tensor(p), N_NEW) for p in PROMPTS]


def test_lock_step_serves_like_one_rank_with_equal_forward_counts(tmp_path):
    rep = _run("lockstep", 3, tmp_path)
    assert [r["tokens"] for r in rep[0]["results"]] == _expected()
    assert rep[0]["health"] == "ok" and rep[0]["ping"] is True
    c = rep[0]["census"]
    assert c["lockstep"] and c["lanes_per_rank"] == 2 and sum(c["per_rank_opened"]) == 6
    assert min(c["per_rank_opened"]) >= 1                      # the requests were spread over the ranks
    counts = [rep[0]["forwards"]] + [r["forwards"] for r in rep[1:]]
    assert len(set(counts)) == 1 and counts[0] > 6, counts      # every verb ran one forward pass on every rank
    assert all(r["filler"] > 0 for r in rep[1:])                # idle ranks filled in with their scratch lane
    # every rank was told the same token bound for the same step, and it covers what the ranks ran together
    assert rep[0]["bounds"] == rep[1]["bounds"] == rep[2]["bounds"] and all(b >= 3 for b in rep[0]["bounds"])
    for r in rep[1:]:
        assert r["loop"] == "stopped" and r["lanes_left"] == 0 and r["free_lanes"] == 2    # only the scratch lane is held


def test_without_lock_step_idle_ranks_skip(tmp_path):
    rep = _run("free", 2, tmp_path)
    assert [r["tokens"] for r in rep[0]["results"]] == _expected()
    assert rep[0]["census"]["lockstep"] is False and rep[0]["census"]["lanes_per_rank"] == 3
    assert rep[1]["filler"] == 0 and rep[1]["free_lanes"] == 3
    assert rep[0]["forwards"] != rep[1]["forwards"] or rep[0]["forwards"] > 0


def test_owner_that_refuses_a_lane_fails_that_request_only(tmp_path):
    rep = _run("open_fault", 3, tmp_path)
    res = rep[0]["results"]
    failed = [r for r in res if r["reason"] == "error"]
    assert len(failed) == 1 and "rank 1 could not open the lane" in failed[0]["error"]
    want = _expected()
    ok = [r["tokens"] for r in res if r["reason"] == "length"]
    assert len(ok) == 5 and all(t in want for t in ok)
    assert rep[0]["health"] == "ok"
    for r in rep[1:]:
        assert r["loop"] == "stopped" and r["lanes_left"] == 0


def test_rank_that_leaves_fails_the_engine_by_time_out(tmp_path):
    rep = _run("leave", 3, tmp_path)
    assert rep[2]["left_after_decode_rounds"] == 2
    assert any(r["reason"] == "error" and "stopped answering" in r.get("error", "") for r in rep[0]["results"])
    assert rep[0]["health"] == "failed" and rep[1]["loop"] == "channel_failed"
