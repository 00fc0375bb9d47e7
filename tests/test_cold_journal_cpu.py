"""The disk tier's journal: framing, torn tails, releases, adoption after a restart, the read-or-prefill verdict."""
import os

import pytest

from ninfer_fusion_b200.runtime.cold_journal import (ColdJournal, RecallCost, SpillRecord, read_frames, token_digest)
from ninfer_fusion_b200.runtime.engine import Engine, RequestOptions


def _file(d, name, n):
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, name), "wb") as f:
        f.write(b"x" * n)


def test_records_replay_and_a_torn_tail_is_ignored_then_truncated(tmp_path):
    d = str(tmp_path)
    j = ColdJournal(d, "fp")
    _file(d, "ckpt_a.pt", 100), _file(d, "ckpt_b.pt", 200), _file(d, "ckpt_c.pt", 300)
    for name, n in (("ckpt_a.pt", 100), ("ckpt_b.pt", 200), ("ckpt_c.pt", 300)):
        assert j.spill(SpillRecord(name, n * 10, n, "s", "turn", [1, 2, 3, n]))
    assert j.release("ckpt_b.pt", "promoted") and not j.release("ckpt_b.pt")
    j.close()
    size = os.path.getsize(j.path)
    with open(j.path, "ab") as f:                       # a crash in the middle of the next record
        f.write(b"\x43\x4c\x4a\x31\xff\x00\x00\x00garbage")
    k = ColdJournal(d, "fp")
    assert sorted(k.live) == ["ckpt_a.pt", "ckpt_c.pt"] and k.report.records == 4 and k.report.released == 1
    assert k.report.ignored_tail_bytes == os.path.getsize(j.path) - size and k.report.valid_bytes == size
    assert k.live["ckpt_c.pt"].tokens == [1, 2, 3, 300] and k.live["ckpt_c.pt"].digest == token_digest([1, 2, 3, 300])
    assert k.spill(SpillRecord("ckpt_d.pt", 1, 1, "s", "turn", [9]))      # appending first cuts the torn tail off
    k.close()
    frames, valid, ignored = read_frames(j.path)
    assert ignored == 0 and frames[-1]["file"] == "ckpt_d.pt" and frames[0] == {"op": "open", "fingerprint": "fp"}
    # a flipped byte inside a record ends the replay there (the records after it are not trusted)
    data = bytearray(open(j.path, "rb").read())
    data[40] ^= 0x55
    open(j.path, "wb").write(bytes(data))
    assert ColdJournal(d, "fp").report.ignored_tail_bytes > 0


def test_another_fingerprint_refuses_the_whole_journal_and_holes_are_released(tmp_path):
    d = str(tmp_path)
    j = ColdJournal(d, "model-a", flush="fsync")
    _file(d, "ckpt_a.pt", 64), _file(d, "ckpt_short.pt", 10)
    j.spill(SpillRecord("ckpt_a.pt", 640, 64, "s", "turn", [1, 2]))
    j.spill(SpillRecord("ckpt_gone.pt", 640, 64, "s", "turn", [1, 2, 3]))
    j.spill(SpillRecord("ckpt_short.pt", 640, 64, "s", "turn", [1, 2, 3, 4]))
    j.spill(SpillRecord("../escape.pt", 1, 1, "s", "turn", [1]))
    j.close()
    other = ColdJournal(d, "model-b")
    assert other.report.refused and not other.live
    mine = ColdJournal(d, "model-a")
    assert "../escape.pt" not in mine.live                 # a record never points outside the directory
    good, holes = mine.adoptable()
    assert [r.file for r in good] == ["ckpt_a.pt"] and sorted(h[0] for h in holes) == ["ckpt_gone.pt", "ckpt_short.pt"]
    assert sorted(mine.live) == ["ckpt_a.pt"] and mine.orphans() == ["ckpt_short.pt"]
    saved = mine.compact()
    assert saved > 0 and sorted(ColdJournal(d, "model-a").live) == ["ckpt_a.pt"]
    with pytest.raises(ValueError):
        ColdJournal(d, "model-a", flush="sometimes")
    # writing through a refused journal starts a new one
    other.spill(SpillRecord("ckpt_n.pt", 1, 1, "s", "turn", [5]))
    other.close()
    assert ColdJournal(d, "model-a").report.refused and sorted(ColdJournal(d, "model-b").live) == ["ckpt_n.pt"]


def test_recall_cost_prefers_prefill_when_the_disk_is_slow():
    fast = RecallCost(read_gbs=7.0, prefill_tok_s=30000.0)
    slow = RecallCost(read_gbs=0.2, prefill_tok_s=30000.0)
    nbytes, n = 32768 * 8192, 8192                     # fp8 KV of an 8k-token frontier, 32 KiB per token
    assert fast.worthwhile(nbytes, n) and not slow.worthwhile(nbytes, n)
    assert fast.read_ms(nbytes) == pytest.approx(nbytes / 7e9 * 1e3 + 1.0) and fast.prefill_ms(n) == pytest.approx(8192 / 30.0)
    assert "-> read" in fast.line(nbytes, n) and "-> prefill" in slow.line(nbytes, n)
    assert fast.decisions == {"read": 1, "prefill": 0} and slow.decisions == {"read": 0, "prefill": 1}
    assert not fast.worthwhile(1 << 20, 8)             # a tiny frontier: the fixed overhead loses to 8 tokens of prefill


def test_frontiers_on_disk_survive_a_restart_of_the_engine(tmp_path):
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.program import ReferenceProgram
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=5, std=0.05)
    reports = []

    def factory(weights_id="w1"):
        def make():
            p = ReferenceProgram(cfg, w, max_lanes=2, max_context=256)
            p.max_checkpoints, p.host_budget_bytes, p.disk_budget_bytes = 2, 1, 1 << 30
            p.cold_dir = str(tmp_path / "cold")
            reports.append(p.enable_cold_journal(weights_id=weights_id, flush="flush"))
            return p
        return make
    first = {}
    eng = Engine(factory(), prefill_chunk=32)
    try:
        for s in range(4):
            prompt = list(range(10 + s, 50 + s))
            first[s] = (prompt, eng.submit(prompt, RequestOptions(max_tokens=4, session=f"s{s}")).wait(timeout=60))
        prog = eng.program
        on_disk = [c for c in prog.checkpoints if c.tier == "disk"]
        assert on_disk and len(prog.cold_journal.live) == len(on_disk)
        assert all(os.path.exists(c.handle["path"]) for c in on_disk)
        s0_on_disk = [c for c in on_disk if c.session == "s0"]
        assert s0_on_disk
    finally:
        eng.shutdown()
    eng.program.cold_journal.close()
    assert reports[0]["adopted"] == 0
    # ---- "restart": a new process would build a new Program over the same directory ----
    eng2 = Engine(factory(), prefill_chunk=32)
    try:
        rep = reports[-1]
        assert rep["adopted"] == len(on_disk) and not rep["holes"] and not rep["refused"] and rep["orphans_removed"] == 0
        prog2 = eng2.program
        assert [c.tier for c in prog2.checkpoints].count("disk") == len(on_disk) and prog2.census()["cold_stats"]["adopted"] == len(on_disk)
        prompt, out = first[0]
        follow = prompt + out + [5, 6, 7]
        cold_run = eng2.submit(follow, RequestOptions(max_tokens=4)).wait(timeout=60)          # no session: no reuse
        hits = eng2.stats.prefix_hits
        warm_run = eng2.submit(follow, RequestOptions(max_tokens=4, session="s0")).wait(timeout=60)
        assert warm_run == cold_run and eng2.stats.prefix_hits == hits + 1 and prog2.cold_stats["promoted"] >= 1
        # the promoted frontier's file is gone and released in the journal
        assert len(prog2.cold_journal.live) < len(on_disk) or prog2.cold_stats["demoted_disk"] >= 1
    finally:
        eng2.shutdown()
    eng2.program.cold_journal.close()
    # ---- other weights: nothing is adopted, the old files are swept as orphans ----
    p3 = factory("w2")()
    assert reports[-1]["refused"] and reports[-1]["adopted"] == 0 and not [c for c in p3.checkpoints if c.tier == "disk"]
    assert not [n for n in os.listdir(str(tmp_path / "cold")) if n.startswith("ckpt_")]


def test_a_damaged_cold_file_costs_the_frontier_not_the_request(tmp_path):
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.cold_journal import RecallCost
    from ninfer_fusion_b200.runtime.program import ReferenceProgram
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=5, std=0.05)
    p = ReferenceProgram(cfg, w, max_lanes=2, max_context=256)
    p.max_checkpoints, p.host_budget_bytes, p.disk_budget_bytes, p.cold_dir = 1, 1, 1 << 30, str(tmp_path / "cold")
    p.enable_cold_journal()
    eng = Engine(lambda: p, prefill_chunk=32)
    try:
        outs = {}
        for s in range(3):
            prompt = list(range(20 + s, 60 + s))
            outs[s] = (prompt, eng.submit(prompt, RequestOptions(max_tokens=3, session=f"s{s}")).wait(timeout=60))
        disk = [c for c in p.checkpoints if c.tier == "disk"]
        assert disk
        victim = max(disk, key=lambda c: len(c.tokens))
        with open(victim.handle["path"], "wb") as f:
            f.write(b"not a checkpoint")
        sess = int(victim.session[1:])
        prompt, out = outs[sess]
        follow = (victim.tokens + [3, 4, 5])[:]
        got = eng.submit(follow, RequestOptions(max_tokens=3, session=victim.session)).wait(timeout=60)
        assert len(got) == 3 and p.cold_stats.get("read_failed", 0) >= 1 and victim not in p.checkpoints
        # a verdict that says "prefill" leaves the frontier on disk and the request still runs
        p.recall_cost = RecallCost(read_gbs=1e-6)
        rest = [c for c in p.checkpoints if c.tier == "disk"]
        if rest:
            c = rest[0]
            got = eng.submit(c.tokens + [7, 8], RequestOptions(max_tokens=2, session=c.session)).wait(timeout=60)
            assert len(got) == 2 and p.recall_cost.decisions["prefill"] >= 1
    finally:
        eng.shutdown()


def test_a_closed_journal_continues_where_it_stopped(tmp_path):
    d = str(tmp_path)
    j = ColdJournal(d, "fp")
    j.spill(SpillRecord("ckpt_a.pt", 1, 1, "s", "turn", [1]))
    j.close()
    j.spill(SpillRecord("ckpt_b.pt", 1, 1, "s", "turn", [2]))
    j.close()
    assert sorted(ColdJournal(d, "fp").live) == ["ckpt_a.pt", "ckpt_b.pt"]


def test_cli_flags_enable_the_journal_and_the_verdict(tmp_path, capsys):
    import argparse
    from ninfer_fusion_b200 import cli
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.program import ReferenceProgram
    w = random_weights(TINY_DENSE, "cpu", seed=5, std=0.05)

    def ns(**kw):
        base = dict(cold_policy="disk", cold_host_bytes="0", cold_disk_path=str(tmp_path), cold_disk_bytes="1g", cold_entropy=False,
                    cold_journal=True, cold_journal_flush="flush", cold_read_gbs=3.0, cold_prefill_tok_s=20000.0, artifact=None,
                    model="tiny-dense", seed=5, weights="bf16")
        base.update(kw)
        return argparse.Namespace(**base)
    p = ReferenceProgram(TINY_DENSE, w, max_lanes=2, max_context=128)
    cli.apply_cold_policy(ns(), p)
    assert p.cold_journal is not None and p.cold_journal.flush == "flush" and p.recall_cost.read_gbs == 3.0
    assert "random:tiny-dense:5:bf16" in p.cold_journal.fingerprint and "adopted 0 frontiers" in capsys.readouterr().err
    for bad in (ns(cold_policy="host", cold_host_bytes="1m"), ns(cold_read_gbs=0.0), ns(cold_policy="none", cold_disk_path="", cold_disk_bytes="0")):
        with pytest.raises(SystemExit):
            cli.apply_cold_policy(bad, ReferenceProgram(TINY_DENSE, w, max_lanes=2, max_context=128))
