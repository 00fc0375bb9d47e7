"""Multi-rank engine control plane on CPU ranks (gloo): identical steps on every rank, AND-reduced admission,
a lane refused by one rank fails on all, a rank that leaves turns into an engine-wide failure and a regroup."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.reference_model import ReferenceModel
from ninfer_fusion_b200.models.weights import random_weights

WORKER = os.path.join(os.path.dirname(__file__), "replicated_worker.py")


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
        assert os.path.exists(path), f"rank {r} wrote no report:\n{logs[r][-2000:]}"
        reports.append(json.load(open(path)))
    return reports


def _expected():
    from tests.replicated_worker import CFG, PROMPTS, W  # same weights and prompts as the workers
    ref = ReferenceModel(CFG, W)
    return [ref.generate_greedy(torch.tensor(p), 6) for p in PROMPTS]


def test_three_ranks_serve_like_one(tmp_path):
    rep = _run("plain", 3, tmp_path)
    want = _expected()
    assert [r["tokens"] for r in rep[0]["results"]] == want
    assert rep[0]["health"] == "ok" and rep[0]["ping"] is True
    for r in rep[1:]:
        assert r["loop"] == "stopped" and r["lanes_left"] == 0 and r["free_lanes"] == 3


def test_lane_refused_by_one_rank_fails_on_all_ranks(tmp_path):
    rep = _run("open_fault", 3, tmp_path)
    res = rep[0]["results"]
    failed = [r for r in res if r["reason"] == "error"]
    assert len(failed) == 1 and "rank 1 could not open the lane" in failed[0]["error"]
    want = _expected()
    ok = [r["tokens"] for r in res if r["reason"] == "length"]
    assert len(ok) == 3 and all(t in want for t in ok)
    assert rep[0]["health"] == "ok" and rep[0]["stats"]["open_failures"] == 1
    for r in rep[1:]:
        assert r["loop"] == "stopped" and r["lanes_left"] == 0 and r["free_lanes"] == 3   # nothing leaked anywhere


def test_admission_is_the_and_of_all_ranks(tmp_path):
    rep = _run("veto", 2, tmp_path)
    assert [r["tokens"] for r in rep[0]["results"]] == _expected()
    assert rep[0]["stats"]["admit_vetoes"] == 3


def test_rank_that_leaves_fails_the_engine_and_the_survivors_regroup(tmp_path):
    rep = _run("leave", 3, tmp_path)
    assert rep[2]["left_after_decode_rounds"] == 2
    res = rep[0]["results"]
    assert any(r["reason"] == "error" and "stopped answering" in r.get("error", "") for r in res)
    assert rep[0]["health"] == "failed"
    assert rep[1]["loop"] == "channel_failed"
    assert rep[0]["health_after_recover"] == "ok"
    assert rep[0]["after_recover"] == _expected()[0]
    assert rep[1]["loop_after_regroup"] == "stopped"
