"""KV storage policy planners (CPU): grammars, bit-budget DP, block descent."""
import pytest

from ninfer_fusion_b200.kv.descent import CellMap, DescentConfig, apply_moves, plan_descent_pass
from ninfer_fusion_b200.kv.policy import (build_ladder, format_layer_storage, parse_layer_storage, parse_tier_formats,
                                          solve_bit_budget)


def test_layer_storage_grammar_round_trip():
    t = parse_layer_storage("all:fp8|0-3:bf16|7:nvfp4", 16)
    assert t[:4] == ["bf16"] * 4 and t[7] == "nvfp4" and t[8] == "fp8"
    assert parse_layer_storage(format_layer_storage(t), 16) == t
    assert format_layer_storage(["fp8"] * 5) == "all:fp8"
    for bad in ("all", "0-99:fp8", "3-1:fp8", "all:fp7", "|", "x:bf16"):
        with pytest.raises(ValueError):
            parse_layer_storage(bad, 16)
    tf = parse_tier_formats("hot=bf16,cold=nvfp4")
    assert (tf.hot, tf.tail, tf.cold) == ("bf16", "fp8", "nvfp4")
    with pytest.raises(ValueError):
        parse_tier_formats("warm=fp8")


def test_ladder_bits_follow_page_geometry():
    lad = build_ladder(256, 64)
    assert lad["bf16"].bits_centi == 1600 and lad["int8"].bits_centi == 825
    assert lad["fp8"].bits_centi == 806 and lad["nvfp4"].bits_centi == 450


def test_bit_budget_is_exact_and_monotone():
    n = 16
    plan16 = solve_bit_budget(n, 16.0)
    assert plan16.tiers == ["bf16"] * n and plan16.penalty_milli_total == 0
    prev_pen = 0
    for target in (12.0, 9.0, 8.3, 6.0, 4.5):
        p = solve_bit_budget(n, target)
        assert p.avg_bits <= target + 1e-9
        assert p.penalty_milli_total >= prev_pen
        prev_pen = p.penalty_milli_total
        assert parse_layer_storage(p.spec, n) == p.tiers
        # packing: precision never decreases with depth
        order = {"nvfp4": 0, "fp8": 1, "int8": 2, "bf16": 3}
        ranks = [order[t] for t in p.tiers]
        assert ranks == sorted(ranks)
    p = solve_bit_budget(n, 8.3)
    # brute-force check on a small instance: 4 layers
    lad = build_ladder()
    import itertools
    best = None
    for combo in itertools.product(lad.values(), repeat=4):
        bits = sum(t.bits_centi for t in combo)
        if bits <= 830 * 4:
            pen = sum(t.penalty_milli for t in combo)
            best = pen if best is None else min(best, pen)
    assert solve_bit_budget(4, 8.3).penalty_milli_total == best
    with pytest.raises(ValueError):
        solve_bit_budget(n, 4.0)
    cold = solve_bit_budget(n, 4.0, cold_cap=4, cold_bits_centi=100)
    assert len(cold.cold_layers) >= 2 and cold.cold_layers == list(range(len(cold.cold_layers)))


def test_block_descent_one_rung_per_pass_oldest_first():
    cfg = DescentConfig(min_age_tokens=128, max_cells_per_pass=3, sink_blocks=1)
    cells = CellMap(page_tokens=64, n_layers=2)
    cells.touch(0, 640)   # 10 blocks
    moves = plan_descent_pass(cells, cfg, n_kv_heads=4, head_dim=256)
    assert len(moves) == 3 and all(m.src == "bf16" and m.dst == "fp8" for m in moves)
    assert [m.block for m in moves] == [1, 1, 2] and moves[0].layer == 0 and moves[1].layer == 1
    assert all(m.bytes_freed == 2 * 64 * 4 * 256 * 1600 // 800 - 2 * 64 * 4 * 256 * 806 // 800 for m in moves)
    apply_moves(cells, cfg, moves)
    # young blocks (within 128 tokens of the frontier) and the sink block never move
    for _ in range(50):
        mv = plan_descent_pass(cells, cfg, 4, 256)
        if not mv:
            break
        assert all(m.block >= 1 and (m.block + 1) * 64 + 128 <= 640 for m in mv)
        apply_moves(cells, cfg, mv)
    assert cells.rungs[(0, 0, 0)] == 0 and cells.rungs[(0, 0, 9)] == 0 and cells.rungs[(0, 1, 3)] == 2
    # last rung + allow_cold -> cold moves; trimming forgets cells beyond the frontier
    mv = plan_descent_pass(cells, cfg, 4, 256, allow_cold=True)
    assert mv and all(m.dst == "cold" for m in mv)
    cells.trim(0, 130)
    assert (0, 0, 3) not in cells.rungs and (0, 0, 2) in cells.rungs
    # resident-byte target stops the pass early
    cells2 = CellMap(64, 1)
    cells2.touch(1, 6400)
    tight = DescentConfig(min_age_tokens=0, max_cells_per_pass=1000, target_resident_bytes=10**12)
    assert plan_descent_pass(cells2, tight, 4, 256) == []


def test_hadamard_frame_is_an_equivalent_k_frame():
    from ninfer_fusion_b200.kv.codec_report import run
    from ninfer_fusion_b200.ops import reference as R
    import torch
    c = run()["codecs"]
    # a floating-point codec keeps relative precision per value, so the rotation neither helps nor hurts much (it
    # matters for fixed-point codecs); what must hold is that q.k is preserved and the error stays in the same range
    a, b = c["fp8-e4m3-row+hadamard"], c["fp8-e4m3-row"]
    assert a["mean_abs_err"] < 1.3 * b["mean_abs_err"] and a["max_abs_err"] < 1.3 * b["max_abs_err"]
    H = R.hadamard_matrix(256)
    assert torch.allclose(H @ H.t(), torch.eye(256), atol=1e-5) and torch.equal(H, H.t())


def test_sliding_window_rows_release_their_early_pages():
    """A windowed row keeps a bounded number of pages: the cache behaves like a ring."""
    import torch
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.runtime.kv_cache import PagedKvCache
    P, window = 16, 100
    kv = PagedKvCache(TINY_DENSE, 32, P, 2, 64, "cpu", formats="bf16")
    free0 = kv.pool.free_pages
    peak = 0
    for n in range(1, 900):
        kv.ensure(0, n + 1)
        kv.release_before(0, n, window)
        peak = max(peak, free0 - kv.pool.free_pages)
    assert peak <= (window + 64) // P + 3            # bounded, although 900 tokens need 57 pages
    pages = kv.row_pages[0]
    first_live = next(i for i, p in enumerate(pages) if p >= 0)
    assert first_live * P <= 900 - window and (first_live + 1) * P > 900 + 1 - window - 64 - P
    assert all(int(kv.table_host[0, i]) == -1 for i in range(first_live))
    assert kv.detach_prefix(0, 200) is None           # not a reusable frontier any more
    kv.free_row(0)
    assert kv.pool.free_pages == free0
    assert kv.release_before(1, 500, 0) == 0


def test_kv_auto_relayout_policy_and_loop():
    from ninfer_fusion_b200.serve.kv_auto_relayout import ColdPolicy, KvAutoRelayout, RelayoutConfig
    from ninfer_fusion_b200.kv.policy import build_ladder
    n = 8
    cfg = RelayoutConfig(target_bits=8.5, min_observations=2, ewma=0.5, hysteresis=0.05)
    pol = ColdPolicy(n, cfg)
    energy = [1.0, 5.0, 0.2, 3.0, 0.1, 4.0, 0.3, 2.0]
    pol.observe(energy)
    assert not pol.decide().changed                       # one observation is not enough
    pol.observe(energy)
    d = pol.decide()
    assert d.changed and len(d.tiers) == n
    ladder = build_ladder()
    bits = [ladder[t].bits_centi for t in d.tiers]
    assert sum(bits) <= 850 * n
    # the most energetic layers hold the most precise tiers
    order = sorted(range(n), key=lambda i: -energy[i])
    assert [bits[i] for i in order] == sorted(bits, reverse=True)
    # small fluctuations inside the hysteresis do not reshuffle the layers
    pol.current = list(d.tiers)
    pol.observe([e * (1.02 if i % 2 else 0.98) for i, e in enumerate(energy)])
    assert not pol.decide().changed

    class FakeEngine:
        def __init__(self):
            self.reloads, self.fail = [], False

        def reload_kv_storage(self, factory, timeout_s=60.0):
            if self.fail:
                raise TimeoutError("busy")
            self.reloads.append(factory())

    eng = FakeEngine()
    samples = iter([None, energy, energy, energy])
    loop = KvAutoRelayout(eng, n, lambda: next(samples), lambda tiers: (lambda: tuple(tiers)), cfg)
    assert not loop.tick().changed and not loop.tick().changed
    d = loop.tick()
    assert d.changed and d.applied and eng.reloads == [tuple(d.tiers)] and loop.policy.current == d.tiers
    assert not loop.tick().changed                        # same statistics, same layout: nothing to do
    eng.fail = True
    loop.policy.current = ["bf16"] * n
    samples = iter([energy])
    d = loop.tick()
    assert d.changed and not d.applied and "drain" in d.reason and loop.policy.current == ["bf16"] * n


def test_mixed_layer_cells_follow_logical_pages_on_cpu():
    """Bookkeeping of a mixed-precision layer (no kernels involved): every logical page gets a hot-tier cell in
    every mixed layer, shared pages keep theirs until the last reference goes, a copy lands in the source's tier,
    and running out of hot cells is a MemoryError that leaves nothing half-allocated."""
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.runtime.kv_cache import CELL_TIER_SHIFT, MixedKvPlanes, PagedKvCache
    kv = PagedKvCache(TINY_DENSE, 16, 16, 3, 8, "cpu", formats="mixed", mixed_capacity=(6, 8, 8))
    L = kv.layers[0]
    assert isinstance(L, MixedKvPlanes) and L.desc.numel() == 13 and kv.mixed == [L]
    kv.ensure(0, 70)                               # five pages
    assert kv.tier_census() == {"bf16": 5, "fp8": 0, "nvfp4": 0}
    assert [L.tier_of(p) for p in kv.row_pages[0]] == [0] * 5
    assert kv.bytes_in_use() == 5 * L.cell_bytes[0]
    kv.fork_row(0, 1, 40)                          # two full pages shared, the partial third one copied
    assert kv.tier_census()["bf16"] == 6 and kv.row_pages[1][:2] == kv.row_pages[0][:2]
    with pytest.raises(MemoryError):
        kv.ensure(2, 16)                           # no hot cell left: the logical page must not leak either
    assert kv.pool.free_pages == 16 - 6 and kv.tier_census()["bf16"] == 6
    kv.free_row(0)                                 # the shared pages stay alive through row 1
    assert kv.tier_census()["bf16"] == 3
    kv.free_row(1)
    assert kv.tier_census() == {"bf16": 0, "fp8": 0, "nvfp4": 0} and kv.pool.free_pages == 16
    assert int(L.cell_map_host.max()) == -1
    # a cell that sits in a colder tier is copied into the same tier
    kv.ensure(0, 20)
    p0 = kv.row_pages[0][0]
    L.free_cell(p0)
    L.alloc_cell(p0, 2)
    kv.fork_row(0, 1, 8)                           # partial first page: copied
    assert L.tier_of(kv.row_pages[1][0]) == 2 and (int(L.cell_map_host[kv.row_pages[1][0]]) >> CELL_TIER_SHIFT) == 2


def test_cyclic_cache_keeps_a_bounded_ring_of_pages_per_row():
    """A windowed row grows without bound in positions while holding a bounded number of pages; pages that slid out
    of the window are unmapped (-1) and their physical pages come back for the new positions."""
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.runtime.kv_cache import CyclicKvCache
    P, W = 16, 64
    kv = CyclicKvCache(TINY_DENSE, W, P, max_rows=2, max_context=4096, device="cpu", formats="bf16", slack=16, n_layers=1)
    assert kv.n_pages == 2 * kv.ring_pages and kv.ring_pages == (64 + 16 + 15) // 16 + 2
    seen = set()
    for n in range(1, 3000, 37):
        kv.ensure(0, n)
        kv.ensure(1, max(1, n // 2))
        assert kv.live_pages(0) <= kv.ring_pages
        seen.update(p for p in kv.row_pages[0] if p >= 0)
        first_visible = max(0, n - W)
        for pos in range(first_visible, n):               # every position the window can see is mapped
            assert kv.table_host[0, pos // P] >= 0
    assert len(seen) <= kv.n_pages                           # 3000 positions went through at most the pool's pages
    assert int((kv.table_host[0] >= 0).sum()) == kv.live_pages(0) <= kv.ring_pages
    assert kv.table_host[0, 0] == -1                         # the oldest page is gone
    kv.free_row(0)
    kv.free_row(1)
    assert kv.pool.free_pages == kv.n_pages


def test_tier_formats_shape_the_per_cell_ladder_and_the_descent_floor():
    from ninfer_fusion_b200.kv.descent import CellMap, DescentConfig, plan_descent_pass
    from ninfer_fusion_b200.kv.policy import parse_tier_formats, tier_formats_on_ladder
    assert tier_formats_on_ladder(parse_tier_formats("")) == (0, "nvfp4")
    assert tier_formats_on_ladder(parse_tier_formats("hot=fp8,tail=fp8,cold=nvfp4")) == (1, "nvfp4")
    assert tier_formats_on_ladder(parse_tier_formats("hot=bf16,tail=fp8,cold=fp8")) == (0, "fp8")
    for bad in ("hot=fp8,tail=bf16", "hot=nvfp4,tail=fp8,cold=fp8", "hot=int8"):
        with pytest.raises(ValueError):
            tier_formats_on_ladder(parse_tier_formats(bad))
    cells = CellMap(64, 1)
    cells.frontier[0] = 64 * 12
    for b in range(12):
        cells.rungs[(0, 0, b)] = 1 if b < 6 else 0          # old blocks already at fp8, newer ones at bf16
    free = plan_descent_pass(cells, DescentConfig(min_age_tokens=64), 2, 256)
    floor = plan_descent_pass(cells, DescentConfig(min_age_tokens=64, floor="fp8"), 2, 256)
    assert any(m.dst == "nvfp4" for m in free)
    assert floor and all(m.dst == "fp8" for m in floor)     # nothing goes below the floor
    with pytest.raises(ValueError):
        plan_descent_pass(cells, DescentConfig(floor="int8"), 2, 256)


def test_relayout_knapsack_assignment_follows_energy_and_allowed_sets():
    from ninfer_fusion_b200.serve.kv_auto_relayout import ColdPolicy, RelayoutConfig
    cfg = RelayoutConfig(target_bits=6.5, min_observations=1, assignment="knapsack",
                         allowed=[None, None, None, ["bf16", "fp8", "int8"], None, None, None, None])
    pol = ColdPolicy(8, cfg, initial=["fp8"] * 8)
    pol.observe([1, 1, 1, 1, 1, 1, 9, 1])
    d = pol.decide()
    order = {"nvfp4": 0, "fp8": 1, "int8": 2, "bf16": 3}
    assert d.changed and order[d.tiers[6]] == max(order[t] for t in d.tiers)      # the energetic layer keeps the precision
    assert d.tiers[3] != "nvfp4"                                                    # a hole the rank assignment cannot express
    ladder_bits = {"bf16": 16.0, "int8": 8.25, "fp8": 8.0625, "nvfp4": 4.5}
    assert sum(ladder_bits[t] for t in d.tiers) / 8 <= 6.5 + 1e-6
    # stability: once applied, a slightly different sample does not trigger another relayout
    pol.current = list(d.tiers)
    pol.observe([1.02, 1, 1, 1, 1, 0.99, 9, 1])
    assert not pol.decide().changed
    with pytest.raises(ValueError):
        ColdPolicy(2, RelayoutConfig(min_observations=0, assignment="greedy")).decide()


def test_stateless_cell_allocation_solve_and_its_named_refusals():
    from ninfer_fusion_b200.kv import descent as D
    cfg = D.DescentConfig(min_age_tokens=64, sink_blocks=1)
    cells = D.CellMap(64, 2)
    cells.touch(0, 64 * 10)                       # one sequence, 10 blocks, 2 layers, all at bf16
    H, Dh = 2, 256
    per = [D.cell_bytes(D.build_ladder(Dh)[n], 64, H, Dh) for n in cfg.ladder]
    full = 20 * per[0]
    table = D.CellCostTable((0.0, 0.01, 0.08), floor_nats=1.0, floor_measured=True)
    # no pressure: the status quo, nothing spent
    a = D.solve_cell_allocation(cells, cfg, full, table, H, Dh)
    assert a.outcome == D.NO_PRESSURE and a.target == cells.rungs
    # a budget reachable with first steps only: every cheap step (bf16 -> fp8) is taken before any expensive one,
    # oldest blocks first among equals, the sink block and the newest block untouched
    budget = full - 6 * (per[0] - per[1])
    a = D.solve_cell_allocation(cells, cfg, budget, table, H, Dh)
    assert a.outcome == D.SOLVED and a.resident_bytes <= budget and a.cells_demoted == 6
    assert all(r <= 1 for r in a.target.values()) and a.spent_nats == pytest.approx(0.06)
    moved = sorted(k for k, r in a.target.items() if r == 1)
    assert {k[2] for k in moved} == {1, 2, 3} and all(a.target[(0, l, 0)] == 0 and a.target[(0, l, 9)] == 0 for l in (0, 1))
    # a deeper budget takes cells down two rungs in ONE solve (no one-rung-per-pass rule: nothing iterates)
    deep = D.solve_cell_allocation(cells, cfg, full // 2, D.CellCostTable((0.0, 0.01, 0.08), 5.0, True), H, Dh)
    assert deep.outcome == D.SOLVED and max(deep.target.values()) == 2 and deep.resident_bytes <= full // 2
    # the device still re-encodes rung by rung: one pass of moves toward the solved allocation, oldest first
    mv = D.moves_toward(cells, cfg, deep, H, Dh)
    assert mv and all(m.src == "bf16" and m.dst == "fp8" for m in mv) and [m.block for m in mv] == sorted(m.block for m in mv)
    D.apply_moves(cells, cfg, mv)
    again = D.solve_cell_allocation(cells, cfg, full // 2, D.CellCostTable((0.0, 0.01, 0.08), 5.0, True), H, Dh)
    assert again.outcome == D.SOLVED                                   # re-solved from the new state, no carry needed
    # the floor is the one quality constraint: a budget that needs more loss than the floor allows is refused by name
    tight = D.solve_cell_allocation(cells, cfg, full // 4, D.CellCostTable((0.0, 0.01, 0.08), 0.05, True), H, Dh)
    assert tight.outcome == D.REFUSED_BUDGET_UNREACHABLE and tight.deficit_bytes > 0 and tight.target == cells.rungs
    unmeasured = D.solve_cell_allocation(cells, cfg, full // 2, D.CellCostTable((0.0, 0.01, 0.08), 5.0, False), H, Dh)
    assert unmeasured.outcome == D.REFUSED_FLOOR_UNMEASURED
    assert D.solve_cell_allocation(cells, cfg, full // 2, D.CellCostTable((0.0, 0.01), 5.0, True), H, Dh).outcome == D.REFUSED_BAD_TABLE
    assert D.solve_cell_allocation(D.CellMap(64, 2), cfg, 1, table, H, Dh).outcome == D.REFUSED_EMPTY
    # the descent floor of the tier-format grammar bounds the solve as well
    capped = D.solve_cell_allocation(cells, D.DescentConfig(min_age_tokens=64, floor="fp8"), full * 3 // 4,
                                     D.CellCostTable((0.0, 0.01, 0.08), 5.0, True), H, Dh)
    assert max(capped.target.values()) <= 1


def test_descent_pass_in_solve_mode_moves_toward_the_solved_allocation():
    from ninfer_fusion_b200.kv import descent as D
    H, Dh = 2, 256
    cells = D.CellMap(64, 1)
    cells.touch(0, 64 * 8)
    per0 = D.cell_bytes(D.build_ladder(Dh)["bf16"], 64, H, Dh)
    table = D.CellCostTable((0.0, 0.01, 0.08), 1.0, True)
    cfg = D.DescentConfig(min_age_tokens=64, target_resident_bytes=8 * per0 * 3 // 4, solve_table=table)
    passes = 0
    while True:
        mv = D.plan_descent_pass(cells, cfg, H, Dh)
        if not mv:
            break
        D.apply_moves(cells, cfg, mv)
        passes += 1
        assert passes < 10
    assert D.resident_bytes(cells, cfg, D.build_ladder(Dh), H, Dh) <= cfg.target_resident_bytes and passes >= 1
    # a floor that cannot pay for the target: the pass moves nothing (no silent compromise)
    cells2 = D.CellMap(64, 1)
    cells2.touch(0, 64 * 8)
    stuck = D.DescentConfig(min_age_tokens=64, target_resident_bytes=per0, solve_table=D.CellCostTable((0.0, 0.01, 0.08), 0.02, True))
    assert D.plan_descent_pass(cells2, stuck, H, Dh) == []
