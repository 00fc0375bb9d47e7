"""Worker scheduling: execution choice, service quanta, blocked-head protection with back-fill, page reservations."""
import itertools
import time

import pytest

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.weights import random_weights
from ninfer_fusion_b200.runtime.engine import (BandwidthGovernor, Engine, RequestOptions, resolve_prefill_chunk_mode)
from ninfer_fusion_b200.runtime.program import ReferenceProgram
from ninfer_fusion_b200.runtime.scheduler import (ExecutionAction, Scheduler, ServiceAccount, choose_execution,
                                                   prefill_quanta_for, projected_service_work)

P, D, W = ExecutionAction.PREFILL, ExecutionAction.DECODE, ExecutionAction.WAIT


def test_execution_choice_alternates_holds_and_never_starves_prefill():
    for have_decode, runnable, prev_decode, admitted in itertools.product([False, True], repeat=4):
        a = choose_execution(have_decode, runnable, prev_decode, admitted)
        if not runnable:
            assert a is (D if have_decode else W)
        elif not have_decode:
            assert a is P                                   # no decode lanes: prefill runs whatever the verdict
        else:
            assert a is (P if prev_decode and admitted else D)
    s = Scheduler()
    seq = []
    for _ in range(6):                                      # both runnable, verdict true: strict 1:1 alternation
        a = s.choose(True, True, True)
        s.ran(a)
        seq.append(a)
    assert seq == [P, D, P, D, P, D]
    held = []
    for i in range(6):                                      # verdict false: decode only, and the holds are counted
        a = s.choose(True, True, False)
        s.ran(a)
        held.append(a)
    assert held == [D] * 6 and s.stats["prefill_holds"] >= 5


def test_service_quanta_follow_the_prefill_unit():
    assert [prefill_quanta_for(n, 128) for n in (0, 1, 128, 129, 2048)] == [0, 1, 1, 2, 16]
    assert projected_service_work(2048, 512, 100) == 4 + 100
    acc = ServiceAccount(projected_service_work(2048, 2048, 10), 2048)     # 1 + 10
    acc.reconcile(2048, 256)                                               # the unit shrank before anything ran
    assert acc.remaining == 8 + 10 and acc.unit == 256
    acc.consume(1)
    acc.reconcile(2048 - 256, 2048)                                        # growing back never refunds
    assert acc.remaining == 7 + 10
    # shrinking by u units and subtracting what was charged lands on the same number as pricing the rest afresh
    for total, unit, done in ((1000, 128, 3), (777, 64, 5)):
        assert prefill_quanta_for(total, unit) - done == prefill_quanta_for(total - done * unit, unit)
    with pytest.raises(RuntimeError):
        ServiceAccount(1, 128).consume(2)


def test_protection_freezes_donors_and_borrowers_never_become_donors():
    s = Scheduler()
    s.observe_head(7)
    p = s.protect(7, active=[1, 2])
    assert p.donors == frozenset({1, 2}) and s.stats["protections"] == 1
    assert s.protect(7, active=[1, 2, 9]) is p                      # same head: same protection, donors stay frozen
    assert s.authorize_backfill(9, active=[1, 2], proof=True) and 9 in p.borrowers
    assert not s.authorize_backfill(10, active=[1, 2, 9], proof=False)      # no proof, no admission
    assert s.authorize_backfill(11, active=[2, 9], proof=True)              # one donor still live
    assert not s.authorize_backfill(12, active=[9, 11], proof=True)         # only borrowers left: the head waits for them
    assert not s.authorize_backfill(7, active=[1], proof=True)              # the head does not back-fill itself
    s.observe_head(8)                                                        # the head changed: protection ends
    assert s.protection is None
    p2 = s.protect(8, active=[9, 11])
    assert p2.epoch == p.epoch + 1 and p2.donors == frozenset({9, 11})      # a new epoch may take old borrowers as donors


def test_prefill_chunk_mode_resolution(monkeypatch):
    monkeypatch.delenv("NINFER_FT_BW_GOV", raising=False)
    assert resolve_prefill_chunk_mode() == "dynamic" and resolve_prefill_chunk_mode("manual") == "manual"
    monkeypatch.setenv("NINFER_FT_BW_GOV", "0")
    assert resolve_prefill_chunk_mode() == "manual" and resolve_prefill_chunk_mode("dynamic") == "dynamic"
    monkeypatch.setenv("NINFER_FT_BW_GOV", "yes")
    with pytest.raises(ValueError):
        resolve_prefill_chunk_mode()
    with pytest.raises(ValueError):
        resolve_prefill_chunk_mode("auto")


def test_governor_thins_the_prefill_share_at_the_minimum_unit_and_restores_it_first():
    g = BandwidthGovernor(512, min_unit=128, tolerance=1.5, recover_rounds=2)
    for _ in range(3):
        g.observe(10.0, False)
    for _ in range(2):
        g.observe(30.0, True)
    assert g.unit == 128 and g.share == 1.0
    g.observe(30.0, True)
    g.observe(30.0, True)
    assert g.unit == 128 and g.share == 0.25
    # credit: one prefill unit per four decode rounds at share 0.25
    g.credit = 0.0
    allowed = []
    for _ in range(8):
        g.on_decode_round()
        allowed.append(g.prefill_allowed())
        if allowed[-1]:
            g.charge_prefill()
    assert allowed == [False, False, False, True, False, False, False, True]
    for _ in range(4):
        g.observe(10.0, True)
    assert g.share == 1.0 and g.unit == 128        # the share comes back before the unit
    for _ in range(4):
        g.observe(10.0, True)
    assert g.unit == 512
    off = BandwidthGovernor(512, enabled=False)
    off.credit = 0.0
    assert off.mode == "manual" and off.prefill_allowed()


class PagedReference(ReferenceProgram):
    """The CPU oracle program with a finite page pool: the lanes' cache lengths are its page accounting."""
    PAGE = 16

    def __init__(self, *a, total_pages: int = 10, **kw):
        super().__init__(*a, **kw)
        self.total_pages = total_pages
        self.peak_pages = 0

    def _pages_for(self, n_tokens: int) -> int:
        return (max(0, n_tokens) + self.PAGE - 1) // self.PAGE

    def _pages_held(self, lane) -> int:
        return self._pages_for(lane.n_cached + 1) if lane.n_cached else 0

    def _pages_free(self) -> int:
        used = sum(self._pages_held(l) for l in self.lanes.values())
        self.peak_pages = max(self.peak_pages, used)
        assert used <= self.total_pages, "page pool over-committed"
        return self.total_pages - used

    def _kv_room(self, n_tokens: int) -> bool:
        return self.pages_available() >= self._pages_for(n_tokens)


@pytest.fixture(scope="module")
def tiny():
    return TINY_DENSE, random_weights(TINY_DENSE, "cpu", seed=5, std=0.05)


def test_reservations_prevent_two_requests_from_being_admitted_against_the_same_pages(tiny):
    cfg, w = tiny
    prog = {}

    def factory():
        prog["p"] = PagedReference(cfg, w, max_lanes=4, max_context=256, total_pages=10)
        return prog["p"]
    eng = Engine(factory, prefill_chunk=32)
    try:
        # each request may grow to 96 positions = 6 pages; the pool has 10: without reservations both pass the
        # admission check on an empty pool and the second one runs the pool dry mid-generation
        a = eng.submit(list(range(10, 50)), RequestOptions(max_tokens=56))
        b = eng.submit(list(range(60, 100)), RequestOptions(max_tokens=56))
        assert len(a.wait(timeout=300)) == 56 and len(b.wait(timeout=300)) == 56
        assert b.t_admit >= a.t_done - 1e-3                  # b got its lane only when a had left
        assert prog["p"].peak_pages <= 10 and eng.health()["status"] == "ok"
    finally:
        eng.shutdown()


def test_backfill_past_a_blocked_head_needs_the_programs_proof(tiny):
    cfg, w = tiny
    prog = {}

    def factory():
        prog["p"] = PagedReference(cfg, w, max_lanes=4, max_context=256, total_pages=10)
        return prog["p"]
    eng = Engine(factory, prefill_chunk=32)
    try:
        donor = eng.submit(list(range(10, 42)), RequestOptions(max_tokens=64))           # 96 positions: 6 pages
        time.sleep(0.3)                                                                   # it is active before the rest arrive
        head = eng.submit(list(range(50, 114)), RequestOptions(max_tokens=64))           # 128 positions: 8 pages, blocked
        big = eng.submit(list(range(120, 150)), RequestOptions(max_tokens=34))           # 64 positions: 4 pages -> refused
        small = eng.submit(list(range(200, 220)), RequestOptions(max_tokens=12))         # 32 positions: 2 pages -> back-filled
        for h in (small, donor, head, big):
            h.wait(timeout=300)
        assert small.t_admit < donor.t_done and small.t_admit < head.t_admit             # it overtook the head ...
        assert donor.t_done - 1e-3 <= head.t_admit <= donor.t_done + 0.5                 # ... which got in as soon as its donor left
        assert big.t_admit >= head.t_admit                                               # the refused one kept its place
        st = eng.health()["scheduler"]
        assert st["protections"] >= 1 and st["backfills"] == 1 and st["backfill_refusals"] >= 1
        assert prog["p"].peak_pages <= 10
        assert [len(h.tokens) for h in (donor, head, big, small)] == [64, 64, 34, 12]
    finally:
        eng.shutdown()
