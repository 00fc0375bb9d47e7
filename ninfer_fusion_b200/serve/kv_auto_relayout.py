"""KV auto-relayout: per-layer statistics -> smoothed "energy" -> per-layer storage tiers -> `Engine.reload_kv_storage`.

The serving layer watches how much each full-attention layer's cache matters (an energy figure per layer, here the
mean K row scale of the layer's cache: layers whose keys are small contribute little to the logits and tolerate a
coarser codec), smooths it with an EWMA, and every `period_s` re-solves the tier assignment under the configured
bits-per-element budget: the multiset of tiers comes from the bit-budget DP, and the precise tiers go to the layers
with the highest energy.  A new plan is applied only when it differs from the running one and the engine can drain.

Reference: src/serve/kv_auto_relayout.{h,cpp} and src/serve/kv_cold_policy.h (energy statistics -> EWMA / quantile
cold policy -> periodic drain + Engine::reload_kv_storage).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..kv.policy import build_ladder, format_layer_storage, solve_bit_budget


@dataclass
class RelayoutConfig:
    target_bits: float = 8.5          # average bits per cached element over the full-attention layers
    period_s: float = 300.0
    ewma: float = 0.2                 # weight of the newest observation
    min_observations: int = 3         # no relayout before this many samples
    hysteresis: float = 0.05          # relative energy margin a layer needs to overtake another (stability)
    drain_timeout_s: float = 30.0
    # how the tiers are spread over the layers: "rank" = the bit-budget allocator's multiset handed out by energy rank
    # (stable under the hysteresis); "knapsack" = the exact per-layer knapsack with every layer's prior penalties
    # scaled by its own energy (kv/adapt_solver.py), which also honours per-layer allowed sets
    assignment: str = "rank"
    allowed: Optional[Sequence[Optional[Sequence[str]]]] = None


@dataclass
class RelayoutDecision:
    spec: str
    tiers: List[str]
    energy: List[float]
    changed: bool
    applied: bool = False
    reason: str = ""


class ColdPolicy:
    """Energy statistics of the layers and the tier assignment that follows from them."""

    def __init__(self, n_layers: int, cfg: RelayoutConfig, initial: Optional[Sequence[str]] = None):
        self.n_layers, self.cfg = n_layers, cfg
        self.energy: List[Optional[float]] = [None] * n_layers
        self.observations = 0
        self.current: List[str] = list(initial) if initial is not None else ["bf16"] * n_layers
        self._rank: List[int] = list(range(n_layers))   # layers by descending energy, kept stable by the hysteresis

    def observe(self, sample: Sequence[float]) -> None:
        if len(sample) != self.n_layers:
            raise ValueError("one energy value per full-attention layer")
        a = self.cfg.ewma
        for i, v in enumerate(sample):
            self.energy[i] = float(v) if self.energy[i] is None else (1 - a) * self.energy[i] + a * float(v)
        self.observations += 1

    def _ranking(self) -> List[int]:
        e = [v or 0.0 for v in self.energy]
        rank = list(self._rank)
        # bubble passes with a margin: a layer moves up only if it beats its neighbour by the hysteresis
        moved = True
        while moved:
            moved = False
            for j in range(len(rank) - 1):
                hi, lo = rank[j], rank[j + 1]
                if e[lo] > e[hi] * (1 + self.cfg.hysteresis):
                    rank[j], rank[j + 1] = lo, hi
                    moved = True
        self._rank = rank
        return rank

    def decide(self) -> RelayoutDecision:
        e = [v or 0.0 for v in self.energy]
        if self.observations < self.cfg.min_observations:
            return RelayoutDecision(format_layer_storage(self.current), list(self.current), e, False,
                                    reason="not enough observations")
        if self.cfg.assignment == "knapsack":
            from ..kv.adapt_solver import solve_for_bits
            mean = sum(e) / max(1, len(e)) or 1.0
            plan = solve_for_bits(self.n_layers, self.cfg.target_bits, [v / mean for v in e], self.cfg.allowed)
            keep = (plan.tiers != self.current and self._close_call(e, plan.tiers))
            tiers = list(self.current) if keep else list(plan.tiers)
            return RelayoutDecision(format_layer_storage(tiers), tiers, e, tiers != self.current,
                                    reason="within the hysteresis of the current layout" if keep else "")
        if self.cfg.assignment != "rank":
            raise ValueError(f"unknown relayout assignment '{self.cfg.assignment}' (rank | knapsack)")
        plan = solve_bit_budget(self.n_layers, self.cfg.target_bits)
        ladder = build_ladder()
        multiset = sorted((t for t in plan.tiers if t != "cold"), key=lambda n: -ladder[n].bits_centi)   # precise first
        multiset += ["nvfp4"] * (self.n_layers - len(multiset))
        tiers = [""] * self.n_layers
        for tier, layer in zip(multiset, self._ranking()):
            tiers[layer] = tier
        return RelayoutDecision(format_layer_storage(tiers), tiers, e, tiers != self.current)


    def _close_call(self, energy: Sequence[float], proposed: Sequence[str]) -> bool:
        """Knapsack mode's stability rule: keep the current layout when it is feasible and its energy-weighted penalty is
        within the hysteresis of the proposed one (a relayout drains the lanes; a marginal gain does not pay for it)."""
        ladder = build_ladder()
        if any(t not in ladder for t in self.current):
            return False
        bits = sum(ladder[t].bits_centi for t in self.current) / 100.0 / self.n_layers
        if bits > self.cfg.target_bits + 1e-9:
            return False

        def cost(tiers):
            return sum(v * ladder[t].penalty_milli for v, t in zip(energy, tiers))
        return cost(self.current) <= cost(proposed) * (1 + self.cfg.hysteresis)


class KvAutoRelayout:
    """Background loop: sample -> policy -> reload.  `sample()` returns one energy value per full-attention layer (or
    None when nothing is cached yet); `make_factory(tiers)` builds the Program factory for a tier list."""

    def __init__(self, engine, n_layers: int, sample: Callable[[], Optional[Sequence[float]]],
                 make_factory: Callable[[List[str]], Callable[[], object]], cfg: Optional[RelayoutConfig] = None,
                 initial: Optional[Sequence[str]] = None, log: Optional[Callable[[dict], None]] = None):
        self.engine, self.sample, self.make_factory = engine, sample, make_factory
        self.cfg = cfg or RelayoutConfig()
        self.policy = ColdPolicy(n_layers, self.cfg, initial)
        self.log = log
        self.history: List[RelayoutDecision] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def tick(self) -> RelayoutDecision:
        s = self.sample()
        if s is not None:
            self.policy.observe(s)
        d = self.policy.decide()
        if d.changed:
            try:
                self.engine.reload_kv_storage(self.make_factory(d.tiers), timeout_s=self.cfg.drain_timeout_s)
                self.policy.current = list(d.tiers)
                d.applied = True
            except TimeoutError:
                d.reason = "engine did not drain; keeping the running layout"
        self.history.append(d)
        if self.log is not None:
            self.log({"event": "kv_relayout", "spec": d.spec, "changed": d.changed, "applied": d.applied, "reason": d.reason})
        return d

    def start(self) -> None:
        def loop():
            while not self._stop.wait(self.cfg.period_s):
                self.tick()
        self._thread = threading.Thread(target=loop, name="kv-auto-relayout", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)


def kv_scale_energy(kv) -> Optional[List[float]]:
    """Energy sample from a PagedKvCache: mean K row scale of the pages in use, per layer (fp8-row layers), or the
    mean |k| of a sample of rows (bf16 layers).  None when no page is in use."""
    import torch
    pages = sorted({p for row in kv.row_pages.values() for p in row if p >= 0})
    if not pages:
        return None
    idx = torch.tensor(pages[:256], dtype=torch.long, device=kv.device)
    out = []
    for l in kv.layers:
        if l.k_scales is not None and l.k_scales.shape[-1] == 2:
            out.append(float(l.k_scales.index_select(0, idx).view(torch.float16).float().abs().mean()))
        elif l.k_scales is None:
            out.append(float(l.k_codes.index_select(0, idx).view(torch.bfloat16).float().abs().mean()))
        else:
            out.append(float(l.k_scales.index_select(0, idx).float().mean()))
    return out
