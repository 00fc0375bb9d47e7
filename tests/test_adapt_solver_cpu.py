"""Per-layer KV format knapsack: exactness against brute force, holes in the allowed sets, layer-indexed evidence."""
import itertools
import random

import pytest

from ninfer_fusion_b200.kv import adapt_solver as A
from ninfer_fusion_b200.kv.policy import build_ladder, solve_bit_budget


def _brute(weights, per, budget, allowed=None):
    tiers = list(per)
    best = None
    for combo in itertools.product(tiers, repeat=len(weights)):
        if any(t not in weights[l] or (allowed and allowed[l] is not None and t not in allowed[l]) for l, t in enumerate(combo)):
            continue
        b = sum(per[t] for t in combo)
        if b > budget:
            continue
        w = sum(weights[l][t] for l, t in enumerate(combo))
        if best is None or (w, b) < (best[0], best[1]):
            best = (w, b, combo)
    return best


def test_dp_is_exact_against_brute_force_with_holes_and_layer_weights():
    ladder = build_ladder(256)
    per = A.page_bytes(ladder, 64, 2, 256)
    rng = random.Random(0)
    for trial in range(20):
        n = 5
        scale = [rng.uniform(0.2, 3.0) for _ in range(n)]
        w = A.prior_weights(n, ladder, scale)
        allowed = [None if rng.random() < 0.5 else rng.sample(list(per), 2) for _ in range(n)]
        budget = rng.randint(n * min(per.values()), n * max(per.values()))
        want = _brute(w, per, budget, allowed)
        if want is None:
            with pytest.raises(A.AdaptInfeasible):
                A.solve(w, per, budget, allowed)
            continue
        got = A.solve(w, per, budget, allowed)
        assert got.weight_total == pytest.approx(want[0]) and got.bytes_total <= budget
        assert all(allowed[l] is None or t in allowed[l] for l, t in enumerate(got.tiers))


def test_holes_are_representable_and_evidence_decides_the_layer():
    # layers 2 and 5 may not take the 4-bit tier: an assignment the prefix-packing allocator cannot produce
    allowed = [None, None, ["bf16", "fp8", "int8"], None, None, ["bf16", "fp8", "int8"], None, None]
    p = A.solve_for_bits(8, 5.5, allowed=allowed)
    assert p.tiers[2] != "nvfp4" and p.tiers[5] != "nvfp4" and p.tiers.count("nvfp4") >= 4 and p.avg_bits <= 5.5 + 1e-9
    # the same budget with layer 6 ten times as sensitive: it is the layer that keeps the precision
    flat = A.solve_for_bits(8, 6.5)
    tilted = A.solve_for_bits(8, 6.5, layer_scale=[1, 1, 1, 1, 1, 1, 10, 1])
    order = {"nvfp4": 0, "fp8": 1, "int8": 2, "bf16": 3}
    assert order[tilted.tiers[6]] == max(order[t] for t in tilted.tiers) and tilted.tiers[6] != "nvfp4"
    assert sorted(flat.tiers) == sorted(tilted.tiers) or tilted.weight_total != flat.weight_total
    # with unit scales the optimum value equals the layer-blind allocator's (it is the special case)
    blind = solve_bit_budget(8, 6.5)
    assert flat.weight_total == pytest.approx(blind.penalty_milli_total)
    with pytest.raises(A.AdaptInfeasible, match="at least"):
        A.solve_for_bits(4, 3.0)


def test_cold_is_a_mode_compared_against_the_plan_without_it():
    ladder = build_ladder(256)
    per = A.page_bytes(ladder, 64, 2, 256)
    w = A.prior_weights(6, ladder)
    tight = 6 * per["nvfp4"] - 4096                      # nothing fits without spilling a layer
    plan, cold = A.solve_with_cold_mode(w, per, tight, cold_bytes=per["nvfp4"] // 4, cold_weight=[500] * 6, cold_cap=2)
    assert cold and plan.tiers[0] == "cold" and plan.bytes_total <= tight
    roomy = 6 * per["fp8"]
    plan2, cold2 = A.solve_with_cold_mode(w, per, roomy, cold_bytes=per["nvfp4"] // 4, cold_weight=[500] * 6, cold_cap=2)
    assert not cold2 and "cold" not in plan2.tiers        # cold costs more than it saves here: the plan without it wins
    with pytest.raises(A.AdaptInfeasible):
        A.solve_with_cold_mode(w, per, 100, cold_bytes=64, cold_weight=[1] * 6, cold_cap=1)
