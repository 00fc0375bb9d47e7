"""KV capacity resolver, materialisation planner, cold-tier budget (host-only logic)."""
import pytest

from ninfer_fusion_b200.models.config import QWEN36_27B, TINY_DENSE
from ninfer_fusion_b200.runtime import capacity as C
from ninfer_fusion_b200.runtime import planner as P


def test_page_range_and_explicit_policy():
    assert C.page_range(4096, 8, 64) == (64, 512)
    assert C.page_range(100, 200, 64) == (200, 400)          # many lanes, short contexts: one page per lane
    curve = C.CapacityCurve(64, 512, 1000, 10)
    plan = C.resolve(curve, 64, 4096, explicit_tokens=8192)
    assert (plan.pages, plan.tokens, plan.reserved_bytes, plan.policy) == (128, 8192, 1000 + 64 * 10, "explicit")
    assert C.resolve(curve, 64, 4096, explicit_tokens=8193).pages == 129      # page rounding pads upwards
    with pytest.raises(C.CapacityError, match="below max_context"):
        C.resolve(curve, 64, 4096, explicit_tokens=4000)
    with pytest.raises(C.CapacityError, match="outside"):
        C.resolve(curve, 64, 4096, explicit_tokens=64 * 513)
    assert C.resolve(curve, 64, 4096).pages == 512 and C.resolve(curve, 64, 4096).policy == "full"


def test_automatic_policy_follows_the_affine_curve():
    curve = C.CapacityCurve(64, 512, 1_000_000, 1000)
    assert C.resolve(curve, 64, 4096, free_bytes=1_000_000, headroom_bytes=0).pages == 64
    assert C.resolve(curve, 64, 4096, free_bytes=1_100_500, headroom_bytes=0).pages == 164
    assert C.resolve(curve, 64, 4096, free_bytes=1_100_500, headroom_bytes=50_000).pages == 114
    assert C.resolve(curve, 64, 4096, free_bytes=10**9).pages == 512                          # clipped at M_max
    with pytest.raises(C.CapacityError, match="minimum reservation"):
        C.resolve(curve, 64, 4096, free_bytes=999_999)
    with pytest.raises(C.CapacityError, match="minimum reservation"):
        C.resolve(curve, 64, 4096, free_bytes=1_000_000, headroom_bytes=1)
    single = C.CapacityCurve(64, 64, 500, 7)
    assert C.resolve(single, 64, 4096, free_bytes=10_000).pages == 64


def test_curve_from_the_model_geometry():
    cfg = QWEN36_27B
    per_page = C.kv_page_bytes(cfg, "fp8", 64)
    assert per_page == 16 * 2 * 4 * 64 * (256 + 2)           # 16 attention layers, K and V, 4 kv heads, row + scale
    assert C.kv_page_bytes(cfg, "nvfp4", 64) == 16 * 2 * 4 * 64 * (128 + 16)
    mixed = ["bf16"] * 2 + ["nvfp4"] * 14
    assert C.kv_page_bytes(cfg, mixed, 64) == 2 * 4 * 64 * (2 * 512 + 14 * 144)
    curve = C.build_curve(cfg, "fp8", 64, max_context=131072, max_concurrency=8)
    assert (curve.m_min, curve.m_max, curve.b_step) == (2048, 16384, per_page)
    assert curve.bytes_at(curve.m_max) - curve.bytes_at(curve.m_min) == (16384 - 2048) * per_page
    plan = C.resolve(curve, 64, 131072, free_bytes=100 << 30, headroom_bytes=4 << 30)
    assert curve.m_min < plan.pages <= curve.m_max and plan.reserved_bytes <= 96 << 30
    tp = C.build_curve(cfg, "fp8", 64, 131072, 8, n_kv_heads=1, gdn_v_heads=12)
    assert tp.b_step * 4 == curve.b_step
    with pytest.raises(C.CapacityError):
        C.kv_page_bytes(TINY_DENSE, ["bf16", "bf16"], 16)


def _owners():
    return [P.Owner("old-big", pages=40, tokens=2560, nbytes=40 << 20, hits=0, last_hit_epoch=0),
            P.Owner("hot-small", pages=8, tokens=512, nbytes=8 << 20, hits=9, last_hit_epoch=99),
            P.Owner("shared-sys", pages=16, tokens=1024, nbytes=16 << 20, hits=3, last_hit_epoch=90, shared=True),
            P.Owner("running", pages=64, tokens=4096, nbytes=64 << 20, pinned=True),
            P.Owner("mid", pages=20, tokens=1280, nbytes=20 << 20, hits=1, last_hit_epoch=60)]


def test_planner_prefers_cheap_losses_and_respects_rooms():
    pl = P.MaterializationPlanner(P.PRESETS["b200"])
    plan = pl.plan(_owners(), need_pages=30, host_room_bytes=0, disk_room_bytes=0, epoch=100)
    assert plan.complete and plan.actions["old-big"] == P.DROP and plan.actions["running"] == P.KEEP
    assert plan.actions["hot-small"] == P.KEEP and plan.actions["shared-sys"] == P.KEEP
    # with host room the same frontier is parked instead of dropped, at a lower expected cost
    parked = pl.plan(_owners(), 30, host_room_bytes=64 << 20, disk_room_bytes=0, epoch=100)
    assert parked.actions["old-big"] == P.TO_HOST and parked.host_bytes == 40 << 20
    assert parked.expected_cost_ns < plan.expected_cost_ns
    # host room for one frontier only: the second victim goes to disk
    both = pl.plan(_owners(), 55, host_room_bytes=41 << 20, disk_room_bytes=1 << 30, epoch=100)
    assert both.complete and both.freed_pages >= 55
    assert sorted(a for a in both.actions.values() if a != P.KEEP) == [P.TO_DISK, P.TO_HOST]
    # more than everything movable: incomplete, everything movable given up, the pinned one untouched
    over = pl.plan(_owners(), 500, epoch=100)
    assert not over.complete and over.freed_pages == 84 and over.actions["running"] == P.KEEP
    assert pl.plan(_owners(), 0).freed_pages == 0


def test_best_first_beats_greedy_within_budget():
    """Greedy by cost per page takes the two small frontiers; one mid-size frontier alone is cheaper in total."""
    pl = P.MaterializationPlanner(P.ContextCost("unit", 1000.0, 0.0, 1.0, 1.0, 0.0), max_expansions=500)
    owners = [P.Owner("a", pages=6, tokens=50, nbytes=1, hits=9, last_hit_epoch=10),
              P.Owner("b", pages=6, tokens=55, nbytes=1, hits=9, last_hit_epoch=10),
              P.Owner("c", pages=10, tokens=95, nbytes=1, hits=9, last_hit_epoch=10)]
    plan = pl.plan(owners, need_pages=10, epoch=10)
    assert plan.complete and plan.actions == {"a": P.KEEP, "b": P.KEEP, "c": P.DROP} and plan.expansions > 0
    greedy_only = P.MaterializationPlanner(pl.cost, max_expansions=0).plan(owners, 10, epoch=10)
    assert greedy_only.complete and greedy_only.expected_cost_ns > plan.expected_cost_ns


def test_cold_tier_budget_watermarks():
    b = P.ColdTierBudget.from_bytes(page_bytes=1 << 20, host_bytes=100 << 20, disk_bytes=1 << 30)
    assert (b.host_pages, b.disk_pages, b.spill_start, b.spill_stop) == (100, 1024, 90, 70)
    assert b.spill_count(89, spilling=False) == 0 and b.spill_count(90, False) == 20
    assert b.spill_count(80, spilling=True) == 10 and b.spill_count(70, True) == 0      # hysteresis
    assert b.admits(95, 0, 5) == "host" and b.admits(96, 0, 5) == "disk" and b.admits(96, 1020, 5) == "drop"
    nodisk = P.ColdTierBudget.from_bytes(1 << 20, 10 << 20, 0)
    assert nodisk.spill_count(10, False) == 0 and nodisk.admits(10, 0, 1) == "drop"
    with pytest.raises(ValueError):
        P.ColdTierBudget.from_bytes(0, 1, 1)
    with pytest.raises(ValueError):
        P.ColdTierBudget.from_bytes(1, 1, 1, high=0.5, low=0.6)


def test_program_uses_the_planner_for_its_victim():
    from ninfer_fusion_b200.runtime.program import Checkpoint, ProgramBase, SHARED_SESSION
    p = ProgramBase(TINY_DENSE, max_lanes=2, max_context=64)
    p._clock = 100
    old_long = Checkpoint("s1", "turn", list(range(400)), None, last_used=10)
    recent_short = Checkpoint("s2", "turn", list(range(20)), None, last_used=99, hits=5)
    shared = Checkpoint(SHARED_SESSION, "shared", list(range(50)), None, last_used=5, hits=4)
    assert p._choose_victim([recent_short, shared, old_long]) is old_long        # plain LRU: the oldest PRIVATE frontier
    assert p._choose_victim([shared]) is shared                                  # a shared prefix only when nothing private is left
    p.planner = P.MaterializationPlanner(P.PRESETS["b200"])
    assert p._choose_victim([recent_short, shared, old_long]) is old_long        # cold, unhit: cheapest to lose
