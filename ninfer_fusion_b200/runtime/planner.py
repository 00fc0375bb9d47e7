"""Resource planning under memory pressure: what to give up so that a request can be admitted.

* ``ContextCost``: machine cost presets -- what it costs to get a context of n tokens back by prefilling it again, by
  copying it from pinned host memory, or by reading it from disk (reference: src/runtime/engine/context_cost.{h,cpp}).
* ``MaterializationPlanner``: picks, for a demand of device pages, a degradation target per cached frontier
  (keep / demote to host / demote to disk / drop) that frees enough pages at the least expected future cost.  The
  search is bounded and anytime: a greedy plan exists after one pass, best-first refinement improves it until the
  expansion budget is spent (reference: src/runtime/engine/materialization_planner.h, bounded anytime search over
  degradation targets; retention classes RecentPrivate / shared credit).
* ``ColdTierBudget``: how many pages the host and disk tiers may hold and when spill / write-back starts
  (reference: src/product/kv_cold_tier_budget.h, cold_spill_writeback.h).
"""
from __future__ import annotations

import heapq
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

KEEP, TO_HOST, TO_DISK, DROP = "keep", "host", "disk", "drop"
ACTIONS = (KEEP, TO_HOST, TO_DISK, DROP)


@dataclass(frozen=True)
class ContextCost:
    """Cost model of one hardware class, in nanoseconds."""
    name: str
    prefill_ns_per_token: float          # rebuilding a frontier by running the prompt again
    prefill_fixed_ns: float
    host_gbps: float                     # pinned host <-> device copy rate
    disk_gbps: float                     # cold file read rate
    copy_fixed_ns: float = 20_000.0

    def rebuild_ns(self, tokens: int) -> float:
        return self.prefill_fixed_ns + tokens * self.prefill_ns_per_token

    def host_restore_ns(self, nbytes: int) -> float:
        return self.copy_fixed_ns + nbytes / self.host_gbps

    def disk_restore_ns(self, nbytes: int) -> float:
        return 4 * self.copy_fixed_ns + nbytes / self.disk_gbps + nbytes / self.host_gbps


# prefill rates: 27B-class hybrid, measured TTFT of this engine on one B200 (2048 tokens in ~80-113 ms); the other
# presets scale with their dense bf16 throughput.  Copy rates: PCIe 5 x16 pinned copies and one NVMe drive.
PRESETS: Dict[str, ContextCost] = {
    "b200": ContextCost("b200", 45_000.0, 2_000_000.0, 50.0, 6.0),
    "h100": ContextCost("h100", 110_000.0, 3_000_000.0, 50.0, 6.0),
    "rtx5090": ContextCost("rtx5090", 400_000.0, 5_000_000.0, 25.0, 3.0),
}


@dataclass
class Owner:
    """One cached frontier competing for device pages."""
    key: object
    pages: int                       # device pages it would free
    tokens: int                      # context length it covers (rebuild cost)
    nbytes: int                      # size of its cold copy
    hits: int = 0                    # times it was selected by a request
    last_hit_epoch: int = 0
    shared: bool = False             # shared-prefix frontier: every session may hit it
    pinned: bool = False             # bound to a running request: may not be touched
    tier: str = "gpu"


@dataclass
class Plan:
    actions: Dict[object, str]
    freed_pages: int
    expected_cost_ns: float
    host_bytes: int
    disk_bytes: int
    expansions: int
    complete: bool                   # frees the demanded pages


class MaterializationPlanner:
    def __init__(self, cost: ContextCost, max_expansions: int = 2048, recency_half_life: int = 64,
                 shared_credit: float = 2.0):
        self.cost = cost
        self.max_expansions = max_expansions
        self.half_life = max(1, recency_half_life)
        self.shared_credit = shared_credit

    # probability-like weight that the frontier is asked for again
    def demand(self, o: Owner, epoch: int) -> float:
        age = max(0, epoch - o.last_hit_epoch)
        w = (1.0 + o.hits) * 0.5 ** (age / self.half_life)
        if o.shared:
            w *= self.shared_credit
        return min(1.0, 0.1 * w)

    def action_cost(self, o: Owner, action: str, epoch: int) -> float:
        p = self.demand(o, epoch)
        if action == KEEP:
            return 0.0
        if action == TO_HOST:
            return p * self.cost.host_restore_ns(o.nbytes)
        if action == TO_DISK:
            return p * self.cost.disk_restore_ns(o.nbytes)
        return p * self.cost.rebuild_ns(o.tokens)

    def plan(self, owners: Sequence[Owner], need_pages: int, host_room_bytes: int = 0, disk_room_bytes: int = 0,
             epoch: int = 0) -> Plan:
        """Frees at least `need_pages` device pages from frontiers on the device tier, or reports the best
        incomplete plan (everything movable given up)."""
        movable = [o for o in owners if o.tier == "gpu" and not o.pinned and o.pages > 0]
        actions = {o.key: KEEP for o in owners}
        if need_pages <= 0:
            return Plan(actions, 0, 0.0, 0, 0, 0, True)

        def options(o: Owner, host_left: int, disk_left: int) -> List[Tuple[float, str]]:
            out = [(self.action_cost(o, DROP, epoch), DROP)]
            if o.nbytes <= host_left:
                out.append((self.action_cost(o, TO_HOST, epoch), TO_HOST))
            if o.nbytes <= disk_left:
                out.append((self.action_cost(o, TO_DISK, epoch), TO_DISK))
            return sorted(out)

        # pass 1 (greedy, always available): cheapest cost per freed page first
        order = sorted(movable, key=lambda o: min(c for c, _ in options(o, host_room_bytes, disk_room_bytes)) / o.pages)
        best = self._greedy(order, need_pages, host_room_bytes, disk_room_bytes, options, actions)
        if not best.complete or len(movable) <= 1:
            return best

        # pass 2 (bounded best-first over subsets in that order): node = (cost so far, index, freed, rooms, choices)
        expansions = 0
        heap: List[Tuple[float, int, int, int, int, int, Tuple[Tuple[int, str], ...]]] = [(0.0, 0, 0, 0, host_room_bytes, disk_room_bytes, ())]
        tick = 1
        suffix_pages = [0] * (len(order) + 1)
        for i in range(len(order) - 1, -1, -1):
            suffix_pages[i] = suffix_pages[i + 1] + order[i].pages
        while heap and expansions < self.max_expansions:
            cost, _, i, freed, host_left, disk_left, chosen = heapq.heappop(heap)
            if cost >= best.expected_cost_ns:
                break                                      # best-first: nothing cheaper remains
            if freed >= need_pages:
                acts = dict(actions)
                hb = db = 0
                for idx, a in chosen:
                    acts[order[idx].key] = a
                    hb += order[idx].nbytes if a == TO_HOST else 0
                    db += order[idx].nbytes if a == TO_DISK else 0
                best = Plan(acts, freed, cost, hb, db, expansions, True)
                continue
            if i >= len(order) or freed + suffix_pages[i] < need_pages:
                continue
            expansions += 1
            o = order[i]
            heapq.heappush(heap, (cost, tick, i + 1, freed, host_left, disk_left, chosen)); tick += 1       # keep it
            for c, a in options(o, host_left, disk_left):
                nh = host_left - (o.nbytes if a == TO_HOST else 0)
                nd = disk_left - (o.nbytes if a == TO_DISK else 0)
                heapq.heappush(heap, (cost + c, tick, i + 1, freed + o.pages, nh, nd, chosen + ((i, a),))); tick += 1
        best.expansions = expansions
        return best

    def _greedy(self, order, need_pages, host_left, disk_left, options, actions) -> Plan:
        acts = dict(actions)
        freed, cost, hb, db = 0, 0.0, 0, 0
        for o in order:
            if freed >= need_pages:
                break
            c, a = options(o, host_left, disk_left)[0]
            acts[o.key] = a
            freed += o.pages
            cost += c
            if a == TO_HOST:
                host_left -= o.nbytes; hb += o.nbytes
            elif a == TO_DISK:
                disk_left -= o.nbytes; db += o.nbytes
        return Plan(acts, freed, cost, hb, db, 0, freed >= need_pages)


@dataclass(frozen=True)
class ColdTierBudget:
    """Page budgets of the cold tiers and the watermarks of the spill loop."""
    host_pages: int
    disk_pages: int
    spill_start: int       # host pages in use at which write-back to disk starts
    spill_stop: int        # ... and at which it stops again (hysteresis)

    @classmethod
    def from_bytes(cls, page_bytes: int, host_bytes: int, disk_bytes: int, high: float = 0.9, low: float = 0.7) -> "ColdTierBudget":
        if page_bytes <= 0:
            raise ValueError("page_bytes must be positive")
        if not 0.0 < low < high <= 1.0:
            raise ValueError("watermarks must satisfy 0 < low < high <= 1")
        hp, dp = host_bytes // page_bytes, disk_bytes // page_bytes
        if dp == 0:
            return cls(hp, 0, hp + 1, hp + 1)              # no disk tier: the host tier never spills, it drops
        return cls(hp, dp, max(1, math.ceil(hp * high)), math.floor(hp * low))

    def spill_count(self, host_in_use: int, spilling: bool) -> int:
        """Pages to write back now: none below the start mark (unless a spill is running), down to the stop mark."""
        if self.disk_pages == 0:
            return 0
        if host_in_use >= self.spill_start or (spilling and host_in_use > self.spill_stop):
            return max(0, host_in_use - self.spill_stop)
        return 0

    def admits(self, host_in_use: int, disk_in_use: int, pages: int) -> str:
        """Where `pages` newly retired pages go: "host", "disk" or "drop"."""
        if host_in_use + pages <= self.host_pages:
            return "host"
        if disk_in_use + pages <= self.disk_pages:
            return "disk"
        return "drop"
