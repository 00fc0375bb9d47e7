"""Adaptive draft width: the controller must settle near the width that maximises tokens per millisecond."""
import random

import pytest

from ninfer_fusion_b200.runtime.spec_width import AdaptiveWidth, CostLine


def _simulate(p_by_depth, a, b, max_width=16, rounds=600, batch=4, seed=0, **kw):
    rng = random.Random(seed)
    ctl = AdaptiveWidth(max_width=max_width, **kw)
    tokens = ms = 0.0
    chosen = []
    for r in range(rounds):
        k = ctl.width
        acc = []
        for _ in range(batch):
            m = 0
            while m < k and rng.random() < p_by_depth(m + 1):
                m += 1
            acc.append(m)
        cost = a + b * k + rng.uniform(-0.02, 0.02) * a
        ctl.observe_round(acc, k, cost)
        if r >= rounds // 2:
            tokens += sum(m + 1 for m in acc) / batch
            ms += cost
            chosen.append(k)
    return ctl, tokens / ms, chosen


def _phi(p_by_depth, a, b, k):
    s, n = 1.0, 1.0
    for i in range(1, k + 1):
        s *= p_by_depth(i)
        n += s
    return n / (a + b * k)


@pytest.mark.parametrize("name,p,a,b", [
    ("code-like", lambda i: 0.93 - 0.01 * i, 14.7, 0.9),
    ("hex-like", lambda i: 0.8 - 0.03 * i, 14.7, 0.9),
    ("repetition", lambda i: 0.995, 14.7, 0.9),
    ("no-benefit", lambda i: 0.45, 14.7, 0.9),
    ("expensive-columns", lambda i: 0.85, 6.0, 2.5),
])
def test_controller_settles_near_the_best_ladder_width(name, p, a, b):
    ctl, achieved, chosen = _simulate(p, a, b)
    best = max(_phi(p, a, b, k) for k in ctl.ladder)
    assert achieved >= 0.93 * best, (name, achieved, best, sorted(set(chosen)))
    # and the measured cost line replaced the defaults
    fit = ctl.cost.fit()
    assert fit is not None and abs(fit[1] - b) < 0.35 * b + 0.1 and abs(fit[0] - a) < 0.2 * a


def test_width_recovers_after_a_bad_stretch():
    ctl = AdaptiveWidth(max_width=8, base_ms=10.0, per_column_ms=0.5)
    for _ in range(64):
        ctl.observe_round([0, 0, 0, 0], ctl.width)          # nothing accepted: fall to the first rung
    assert ctl.width == ctl.ladder[0]
    for _ in range(200):
        ctl.observe_round([ctl.width] * 4, ctl.width)       # everything accepted: climb back to the top
    assert ctl.width == ctl.ladder[-1]


def test_observation_is_censored_beyond_the_first_rejection():
    ctl = AdaptiveWidth(max_width=4, cadence=1000)
    ctl.observe_round([1], extent=4)     # draft 1 accepted, draft 2 rejected, drafts 3 and 4 unobserved
    assert ctl.reach[1:] == [1.0, 1.0, 0.0, 0.0] and ctl.accept[1:] == [1.0, 0.0, 0.0, 0.0]
    ctl.observe_round([4], extent=4)     # all four accepted
    assert ctl.reach[4] == 1.0 and ctl.accept[4] == 1.0 and ctl.reach[1] == pytest.approx(1.9)
    p = ctl.hit_rates()
    assert p[0] > 0.9 and p[1] < p[0]


def test_cost_line_needs_two_widths_and_a_physical_fit():
    line = CostLine()
    line.observe(4, 18.0)
    line.observe(4, 18.2)
    assert line.fit() is None                      # one width: slope not identified
    line.observe(8, 21.8)
    a, b = line.fit()
    assert 13.0 < a < 15.5 and 0.8 < b < 1.1
    bad = CostLine()
    bad.observe(2, 30.0)
    bad.observe(6, 10.0)                           # a falling line is noise, not a cost model
    assert bad.fit() is None


def test_ladder_is_clipped_to_the_maximum_width():
    ctl = AdaptiveWidth(max_width=5)
    assert ctl.ladder == (1, 2, 3, 4, 5) and ctl.width in ctl.ladder
    with pytest.raises(ValueError):
        AdaptiveWidth(max_width=0)
