"""Per-layer KV format selection as an exact multiple-choice knapsack.

`policy.solve_bit_budget` minimises a sum of tier penalties under one bit budget; its objective has no layer index, so
WHICH layer gets which tier is decided afterwards by a packing rule.  Here the decision variable is per layer:

    choose T(l) in F_l for every layer l,   minimise  sum_l W[l][T(l)],   subject to  sum_l bytes[T(l)] <= budget

with F_l an arbitrary allowed set per layer (holes are representable: "layers 2 and 5 may not take the 4-bit tier"),
W a per-layer weight matrix (per-layer EVIDENCE has somewhere to live: a measured sensitivity, or key energy times the
tier's prior penalty) and the byte budget on an exact integer grid (plane bytes of a page are multiples of 16, so no
rounding of fractional bits enters the recurrence).  The DP is exact over (layer, bytes / grid); ties prefer fewer
bytes, then the wider tier on the deeper layer.  Cold is a MODE, not a pseudo-tier: `solve_with_cold_mode` runs the
exact DP with and without an admitted cold option and returns the better plan.

Reference: src/product/kv_adapt_solver.h (per-layer allowed sets, layer-indexed objective, 16-byte grid, cold as a
mode), src/product/kv_perlayer_policy.h.
"""
from __future__ import annotations

from dataclasses import dataclass
from math import gcd
from typing import Dict, List, Optional, Sequence, Tuple

from .descent import cell_bytes
from .policy import Tier, build_ladder, format_layer_storage

GRID = 16


@dataclass
class AdaptPlan:
    tiers: List[str]
    spec: str
    bytes_total: int          # per page over all layers
    weight_total: float
    avg_bits: float
    budget_bytes: int


class AdaptInfeasible(ValueError):
    pass


def page_bytes(ladder: Dict[str, Tier], page_tokens: int, n_kv_heads: int, head_dim: int) -> Dict[str, int]:
    return {n: cell_bytes(t, page_tokens, n_kv_heads, head_dim) for n, t in ladder.items() if t.executable}


def prior_weights(n_layers: int, ladder: Dict[str, Tier], layer_scale: Optional[Sequence[float]] = None) -> List[Dict[str, float]]:
    """W[l][tier] = scale_l x the tier's prior penalty (scale 1 everywhere: the layer-blind objective as a special case)."""
    s = list(layer_scale) if layer_scale is not None else [1.0] * n_layers
    if len(s) != n_layers:
        raise ValueError("one scale per layer")
    return [{n: float(s[l]) * t.penalty_milli for n, t in ladder.items() if t.executable} for l in range(n_layers)]


def solve(weights: Sequence[Dict[str, float]], bytes_per_tier: Dict[str, int], budget_bytes: int,
          allowed: Optional[Sequence[Optional[Sequence[str]]]] = None, bits_of: Optional[Dict[str, float]] = None) -> AdaptPlan:
    """Exact DP.  `weights[l]` maps the tiers layer l may take (further narrowed by `allowed[l]`) to their cost."""
    n = len(weights)
    grid = GRID
    for b in bytes_per_tier.values():
        grid = gcd(grid, b) if b % GRID else grid
    cost = {t: b // grid for t, b in bytes_per_tier.items()}
    cap = budget_bytes // grid
    INF = float("inf")
    # best[b] = (weight, choices) using exactly b grid units so far
    best: Dict[int, Tuple[float, Tuple[str, ...]]] = {0: (0.0, ())}
    order = sorted(bytes_per_tier, key=lambda t: -bytes_per_tier[t])     # wider first: stable tie-break
    for l in range(n):
        opts = [t for t in order if t in weights[l] and (allowed is None or allowed[l] is None or t in allowed[l])]
        if not opts:
            raise AdaptInfeasible(f"layer {l} has no allowed tier")
        nxt: Dict[int, Tuple[float, Tuple[str, ...]]] = {}
        for used, (w, path) in best.items():
            for t in opts:
                b = used + cost[t]
                if b > cap:
                    continue
                cand = (w + weights[l][t], path + (t,))
                cur = nxt.get(b)
                if cur is None or cand[0] < cur[0] - 1e-12:
                    nxt[b] = cand
        if not nxt:
            floor = sum(min(cost[t] for t in order if t in weights[k] and (allowed is None or allowed[k] is None or t in allowed[k]))
                        for k in range(n)) * grid
            raise AdaptInfeasible(f"no assignment fits {budget_bytes} bytes per page; the allowed sets need at least {floor}")
        best = nxt
    used, (w, path) = min(best.items(), key=lambda kv: (kv[1][0], kv[0]))
    total = used * grid
    bits = None
    if bits_of is not None:
        bits = sum(bits_of[t] for t in path) / n
    return AdaptPlan(list(path), format_layer_storage(list(path)), total, w, bits if bits is not None else 0.0, budget_bytes)


def solve_for_bits(n_layers: int, target_bits: float, layer_scale: Optional[Sequence[float]] = None,
                   allowed: Optional[Sequence[Optional[Sequence[str]]]] = None, page_tokens: int = 64, n_kv_heads: int = 4,
                   head_dim: int = 256, ladder: Optional[Dict[str, Tier]] = None) -> AdaptPlan:
    """The front-end form: an average-bits ceiling instead of bytes, prior penalties scaled per layer."""
    ladder = ladder or build_ladder(head_dim)
    per = page_bytes(ladder, page_tokens, n_kv_heads, head_dim)
    elems = 2 * page_tokens * n_kv_heads * head_dim
    budget = int(target_bits * elems * n_layers / 8)
    bits = {n: ladder[n].bits_centi / 100.0 for n in per}
    return solve(prior_weights(n_layers, ladder, layer_scale), per, budget, allowed, bits)


def solve_with_cold_mode(weights: Sequence[Dict[str, float]], bytes_per_tier: Dict[str, int], budget_bytes: int,
                         cold_bytes: int, cold_weight: Sequence[float], cold_cap: int,
                         allowed: Optional[Sequence[Optional[Sequence[str]]]] = None) -> Tuple[AdaptPlan, bool]:
    """Cold as a mode: the exact DP without cold, and with up to `cold_cap` of the shallowest layers spilled (each at
    `cold_bytes` resident bytes and its own `cold_weight`); returns (better plan, cold admitted)."""
    plans = []
    try:
        plans.append((solve(weights, bytes_per_tier, budget_bytes, allowed), False))
    except AdaptInfeasible:
        pass
    for k in range(1, min(cold_cap, len(weights)) + 1):
        w2 = [dict(w) for w in weights]
        al = [None if allowed is None else allowed[i] for i in range(len(weights))]
        for l in range(k):
            w2[l] = {"cold": float(cold_weight[l])}
            al[l] = None
        try:
            p = solve(w2, dict(bytes_per_tier, cold=cold_bytes), budget_bytes, al)
            plans.append((p, True))
        except AdaptInfeasible:
            continue
    if not plans:
        raise AdaptInfeasible("no assignment fits the budget, with or without cold layers")
    return min(plans, key=lambda pc: (pc[0].weight_total, pc[0].bytes_total))
