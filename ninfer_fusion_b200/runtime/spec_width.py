"""Adaptive draft width for chained speculative rounds.

A round that drafts k tokens costs C(k) = a + b * k milliseconds (one captured graph per width, so a column that is
not drafted really is not paid for) and emits N(k) = 1 + S_1 + ... + S_k tokens on average, where S_i is the
probability that the first i drafts are all accepted.  Throughput N(k) / C(k) grows with column k exactly while

    S_k >= b * (1 + S_1 + ... + S_{k-1}) / (a + b * (k - 1))

(compare N(k) / C(k) with N(k-1) / C(k-1); the denominator is the cost BEFORE the column is added).  The controller
keeps

  * per depth i a decayed count of rounds that reached depth i and of rounds that accepted draft i.  A round with
    `accepted` of `extent` drafts observes depths 1 .. min(accepted + 1, extent) and says nothing about deeper ones;
    p_i = accept_i / reach_i with a Beta prior whose weight shrinks with the share of rounds that reach depth i
    (otherwise the optimistic prior, not the data, prices the rarely reached depths);
  * a decayed least-squares line through (width, round milliseconds) for a and b, used once two different widths
    have been timed and only inside a physical band;

and every `cadence` rounds picks the widest prefix of columns that all pass the test, snapped down to a ladder of
widths (one graph is captured per ladder width, not per integer).

Reference: src/targets/qwen3_6/impl/runtime/mtp_window_cut.h (criterion, estimator with prior shrinkage, cost
calibration, re-decision cadence), include/ninfer/ops/mtp_round.h:36,126 (width ladder of the captured rounds).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple


@dataclass
class CostLine:
    """Decayed least squares of round time against drafted width."""
    decay: float = 0.9
    w: float = 0.0
    sx: float = 0.0
    sy: float = 0.0
    sxx: float = 0.0
    sxy: float = 0.0
    samples: int = 0
    last: Optional[Tuple[float, float]] = None

    def observe(self, width: float, ms: float) -> None:
        if width <= 0 or ms <= 0:
            return
        d = self.decay
        self.w = self.w * d + 1.0
        self.sx = self.sx * d + width
        self.sy = self.sy * d + ms
        self.sxx = self.sxx * d + width * width
        self.sxy = self.sxy * d + width * ms
        self.samples += 1
        cur = self._solve()
        if cur is not None:
            self.last = cur

    def _solve(self) -> Optional[Tuple[float, float]]:
        den = self.w * self.sxx - self.sx * self.sx
        # the widths inside the decayed window must still spread: once the controller has sat on one width for a
        # while the slope is a ratio of two vanishing numbers, and the last identified line is kept instead
        if self.samples < 2 or den <= 1e-3 * self.w * self.sxx:
            return None
        b = (self.w * self.sxy - self.sx * self.sy) / den
        a = (self.sy - b * self.sx) / self.w
        # a decode round of a model worth drafting for takes 0.2 .. 400 ms, a drafted column 0.01 .. 8 ms
        if not (0.2 <= a <= 400.0 and 0.01 <= b <= 8.0):
            return None
        return a, b

    def fit(self) -> Optional[Tuple[float, float]]:
        """(a, b) in milliseconds: the most recent identified and physical line, None before there is one."""
        return self.last


@dataclass
class AdaptiveWidth:
    max_width: int
    ladder: Sequence[int] = (1, 2, 3, 4, 6, 8, 12, 16)
    base_ms: float = 12.0          # a and b until the cost line is identified
    per_column_ms: float = 0.6
    decay: float = 0.9             # per observed round
    prior_accept: float = 1.8      # Beta prior with mean 0.9: an optimistic cold start drafts wide and learns fast
    prior_reject: float = 0.2
    cadence: int = 8               # rounds between two decisions
    start: Optional[int] = None    # first width (default: the middle of the ladder)
    calibrate: bool = True         # False: keep base_ms / per_column_ms, ignore measured round times
    reach: List[float] = field(default_factory=list)
    accept: List[float] = field(default_factory=list)
    cost: CostLine = field(default_factory=CostLine)
    rounds: int = 0
    trace: List[Tuple[int, int, float]] = field(default_factory=list)   # (round, width, threshold of its last column)

    def __post_init__(self) -> None:
        if self.max_width < 1:
            raise ValueError("max_width must be >= 1")
        rungs = sorted({int(k) for k in self.ladder if 1 <= int(k) <= self.max_width} | {self.max_width})
        self.ladder = tuple(rungs)
        self.reach = [0.0] * (self.max_width + 1)
        self.accept = [0.0] * (self.max_width + 1)
        self.cost.decay = self.decay
        self.width = self.start if self.start in rungs else rungs[len(rungs) // 2]

    # ------------------------------------------------------------------ observations
    def observe_round(self, accepted: Sequence[int], extent: int, ms: Optional[float] = None) -> None:
        """`accepted[b]` drafts of `extent` were accepted for sequence b in a round that took `ms` milliseconds."""
        for i in range(1, self.max_width + 1):
            self.reach[i] *= self.decay
            self.accept[i] *= self.decay
        for m in accepted:
            seen = min(int(m) + 1, extent)
            for i in range(1, seen + 1):
                self.reach[i] += 1.0
                if i <= m:
                    self.accept[i] += 1.0
        if ms is not None and self.calibrate:
            self.cost.observe(float(extent), float(ms))
        self.rounds += 1
        if self.rounds % self.cadence == 0:
            self.width = self.decide()

    # ------------------------------------------------------------------ estimate and decision
    def hit_rates(self) -> List[float]:
        """p_1 .. p_max: depth-conditional acceptance; depths never reached carry the deepest measured value."""
        prior_mean = self.prior_accept / (self.prior_accept + self.prior_reject)
        out, carried = [], prior_mean
        for i in range(1, self.max_width + 1):
            if self.reach[i] > 0.0:
                share = self.reach[i] / self.reach[1] if self.reach[1] > 0.0 else 0.0
                p = (self.accept[i] + self.prior_accept * share) / (self.reach[i] + (self.prior_accept + self.prior_reject) * share)
                carried = p
            else:
                p = carried
            out.append(p)
        return out

    def cost_model(self) -> Tuple[float, float]:
        return self.cost.fit() or (self.base_ms, self.per_column_ms)

    def best_prefix(self) -> Tuple[int, float]:
        """Widest k whose columns 1..k all pass the marginal test, and the threshold the last examined column faced."""
        a, b = self.cost_model()
        survival, tokens, k, thr = 1.0, 1.0, 0, 0.0
        for i, p in enumerate(self.hit_rates(), start=1):
            survival *= p
            thr = b * tokens / (a + b * (i - 1))
            if survival < thr:
                break
            tokens += survival
            k = i
        return k, thr

    def decide(self) -> int:
        k, thr = self.best_prefix()
        width = self.ladder[0]
        for rung in self.ladder:
            if rung <= k:
                width = rung
        self.trace.append((self.rounds, width, thr))
        return width

    def expected_throughput(self, k: int) -> float:
        """Tokens per millisecond the current estimates predict for width k (used by tests and traces)."""
        a, b = self.cost_model()
        s, n = 1.0, 1.0
        for p in self.hit_rates()[:k]:
            s *= p
            n += s
        return n / (a + b * k)
