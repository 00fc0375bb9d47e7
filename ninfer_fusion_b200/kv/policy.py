"""KV-cache storage policy: tier vocabulary, per-layer tables, bit-budget allocation.

Host-only planners (no GPU): the grammar that names a storage tier per full-attention
layer (`all:<tier>` / `A-B:<tier>` clauses joined by `|`), the `hot=,tail=,cold=` tier-format
grammar, and the fractional bit-budget allocator that picks one tier per layer so that the
average bits per KV element stays inside a budget while a quality penalty is minimised
(exact DP over (bits used, cold layers used)).  Behavioural reference:
src/product/kv_options.h (layer-storage grammar), src/kvcfg/kv_formats.h (tier-format grammar),
src/product/kv_bit_budget.h:1-80,369-378 (ladder, DP, packing order).  The ladder here lists the
tiers this engine executes; bits/element come from this engine's own page geometry.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..ops.reference import KV_BF16, KV_FP8_ROW, KV_INT8_GROUP, KV_NVFP4, kv_bits_per_value


@dataclass(frozen=True)
class Tier:
    name: str
    fmt: int
    bits_centi: int      # bits per KV element x 100 (K and V averaged)
    penalty_milli: int   # quality prior x 1000, lower is better
    executable: bool = True


def build_ladder(head_dim: int = 256, int8_group: int = 64) -> Dict[str, Tier]:
    """Tier ladder for a given geometry.  Penalties follow the reference's needle-sweep priors."""
    def bits(fmt):
        return int(round(kv_bits_per_value(fmt, head_dim, int8_group) * 100))
    return {
        "bf16": Tier("bf16", KV_BF16, bits(KV_BF16), 0),
        "int8": Tier("int8", KV_INT8_GROUP, bits(KV_INT8_GROUP), 20),
        "fp8": Tier("fp8", KV_FP8_ROW, bits(KV_FP8_ROW), 30),
        "nvfp4": Tier("nvfp4", KV_NVFP4, bits(KV_NVFP4), 300),
    }


TIER_NAMES = ("bf16", "int8", "fp8", "nvfp4")


# ----------------------------------------------------------------------------- layer-storage grammar
def parse_layer_storage(spec: str, n_layers: int, default: str = "bf16") -> List[str]:
    """`all:fp8|0-3:bf16|7:nvfp4` -> one tier name per full-attention layer (later clauses win)."""
    out = [default] * n_layers
    if not spec:
        return out
    for clause in spec.split("|"):
        clause = clause.strip()
        if not clause:
            raise ValueError("empty clause in layer-storage spec")
        if ":" not in clause:
            raise ValueError(f"clause '{clause}' must look like RANGE:TIER")
        rng, tier = (s.strip() for s in clause.split(":", 1))
        if tier not in TIER_NAMES:
            raise ValueError(f"unknown KV tier '{tier}' (known: {', '.join(TIER_NAMES)})")
        if rng == "all":
            lo, hi = 0, n_layers - 1
        elif "-" in rng:
            a, b = rng.split("-", 1)
            lo, hi = int(a), int(b)
        else:
            lo = hi = int(rng)
        if lo < 0 or hi >= n_layers or lo > hi:
            raise ValueError(f"layer range '{rng}' outside 0..{n_layers - 1}")
        for i in range(lo, hi + 1):
            out[i] = tier
    return out


def format_layer_storage(tiers: Sequence[str]) -> str:
    """Inverse of parse_layer_storage: run-length clauses, `all:` when uniform."""
    if not tiers:
        return ""
    if all(t == tiers[0] for t in tiers):
        return f"all:{tiers[0]}"
    clauses, start = [], 0
    for i in range(1, len(tiers) + 1):
        if i == len(tiers) or tiers[i] != tiers[start]:
            rng = f"{start}" if i - 1 == start else f"{start}-{i - 1}"
            clauses.append(f"{rng}:{tiers[start]}")
            start = i
    return "|".join(clauses)


@dataclass(frozen=True)
class TierFormats:
    """`hot=<tier>,tail=<tier>,cold=<tier>`: recent window, older resident pages, spilled pages."""
    hot: str = "bf16"
    tail: str = "fp8"
    cold: str = "nvfp4"


def parse_tier_formats(spec: str) -> TierFormats:
    vals = {"hot": "bf16", "tail": "fp8", "cold": "nvfp4"}
    if spec:
        for part in spec.split(","):
            if "=" not in part:
                raise ValueError(f"'{part}' must look like role=tier")
            k, v = (s.strip() for s in part.split("=", 1))
            if k not in vals:
                raise ValueError(f"unknown role '{k}' (hot, tail, cold)")
            if v not in TIER_NAMES:
                raise ValueError(f"unknown KV tier '{v}'")
            vals[k] = v
    return TierFormats(**vals)


def tier_formats_on_ladder(tf: TierFormats, ladder: Sequence[str] = ("bf16", "fp8", "nvfp4")) -> Tuple[int, str]:
    """What a `hot=,tail=,cold=` triple means for per-cell tiers on a fixed precision ladder: (index of the tier new
    pages start in, deepest tier a resident cell may descend to).  The three roles must walk DOWN the ladder (a tail
    wider than the hot tier would re-encode upwards) and every role must be a rung of it."""
    for role in ("hot", "tail", "cold"):
        if getattr(tf, role) not in ladder:
            raise ValueError(f"{role}={getattr(tf, role)} is not a tier of the per-cell ladder {'/'.join(ladder)}")
    h, t, c = (ladder.index(getattr(tf, r)) for r in ("hot", "tail", "cold"))
    if not h <= t <= c:
        raise ValueError(f"hot={tf.hot},tail={tf.tail},cold={tf.cold} does not descend the ladder {'/'.join(ladder)}")
    return h, tf.cold


# ----------------------------------------------------------------------------- bit-budget allocator
@dataclass
class BitBudgetPlan:
    tiers: List[str]                 # per full-attention layer ("cold" marks a cold-pool layer)
    bits_centi_total: int
    penalty_milli_total: int
    avg_bits: float
    spec: str                        # packed layer-storage grammar for the hot layers
    cold_layers: List[int] = field(default_factory=list)


def solve_bit_budget(n_layers: int, target_bits: float, ladder: Optional[Dict[str, Tier]] = None,
                     cold_cap: int = 0, cold_bits_centi: int = 0, cold_penalty_milli: int = 500) -> BitBudgetPlan:
    """Minimise the summed penalty subject to sum(bits) <= target_bits * n_layers.

    Exact DP over (layer index, bits used, cold layers used).  Ties prefer fewer bits.  Packing: the
    chosen multiset of tiers is laid out with the LOWEST precision on the shallow layers and the
    highest precision on the deep layers (deep layers keep the hot high-precision tail); cold layers
    take the shallowest block."""
    ladder = ladder or build_ladder()
    tiers = [t for t in ladder.values() if t.executable]
    budget = int(round(target_bits * 100)) * n_layers
    min_bits = min(t.bits_centi for t in tiers)
    if cold_cap <= 0 and min_bits * n_layers > budget:
        raise ValueError(f"budget {target_bits} bits/element is below the smallest tier ({min_bits / 100})")
    INF = 1 << 60
    # state: dict[(bits_used, cold_used)] -> (penalty, choice list)
    states: Dict[Tuple[int, int], Tuple[int, Tuple[str, ...]]] = {(0, 0): (0, ())}
    for _ in range(n_layers):
        nxt: Dict[Tuple[int, int], Tuple[int, Tuple[str, ...]]] = {}
        for (bits, cold), (pen, path) in states.items():
            cands = [(t.bits_centi, t.penalty_milli, t.name, 0) for t in tiers]
            if cold < cold_cap:
                cands.append((cold_bits_centi, cold_penalty_milli, "cold", 1))
            for b, pm, name, dc in cands:
                nb = bits + b
                if nb > budget:
                    continue
                key = (nb, cold + dc)
                val = (pen + pm, path + (name,))
                cur = nxt.get(key)
                if cur is None or val[0] < cur[0]:
                    nxt[key] = val
        if not nxt:
            raise ValueError("no allocation fits the budget")
        states = nxt
    best_key = min(states, key=lambda k: (states[k][0], k[0], k[1]))
    pen, path = states[best_key]
    order = {"cold": -1}
    for t in tiers:
        order[t.name] = t.bits_centi
    packed = sorted(path, key=lambda n: order[n])   # cold first, then ascending precision
    cold_layers = [i for i, n in enumerate(packed) if n == "cold"]
    hot = [n if n != "cold" else "nvfp4" for n in packed]
    return BitBudgetPlan(list(packed), best_key[0], pen, best_key[0] / 100.0 / n_layers,
                         format_layer_storage(hot), cold_layers)
