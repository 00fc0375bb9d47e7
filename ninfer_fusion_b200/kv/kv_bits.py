"""K / V bit ceilings: three entry points over the one bit-budget allocator.

* **joint** -- one ceiling (average bits per KV element) for the whole stack: `policy.solve_bit_budget` picks one tier
  per full-attention layer.  Refuses only a ceiling no tier can reach, and names the cheapest tier.
* **split** -- K has its own ceiling and V has its own; each plane's per-layer layering is solved on its own budget (and
  on its own penalty column when a per-plane score table is given), and the two per-layer vectors are then reconciled
  layer by layer against the (K format, V format) pairs the engine can build.  A layer's pages carry ONE format for both
  planes here, so the buildable pairs are the diagonal; a layer whose two requirements differ is refused BY INDEX with
  the missing cell named, and the refusal carries the deployable joint plan at min(k, v), which honours both ceilings.
  Equal ceilings always reconcile (the two solves are the same solve).
* **ceiling** -- opt-in: deploy the joint plan at min(k, v) and report the headroom of the wider plane that cannot be
  spent.  Never chosen silently.
* **score table** -- the penalty column of the ladder as a table that runs without a model: `show` prints it with its
  provenance (a prior, not a measurement, unless it was loaded from a file), `emit` writes it in the grammar that
  `parse_scores` reads back (`tier=penalty` lines), so a measured table can replace the prior.

A named score table is never dropped: a per-plane table in the joint reading, or a non-joint mode with a single
ceiling, is refused by name instead of being loaded and ignored.

Reference: src/product/kv_kv_bits.h (entries joint / split / score table, refusals, ceiling mode),
src/product/kv_bit_budget.h:738-773 (score-table grammar).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence, Tuple

from .policy import BitBudgetPlan, Tier, build_ladder, format_layer_storage, solve_bit_budget

MIN_BITS, MAX_BITS = 0.01, 16.0

# (K format, V format) -> tier that builds it.  One format drives both planes of a layer's pages.
BUILDABLE_PAIRS: Dict[Tuple[str, str], str] = {(t, t): t for t in ("bf16", "int8", "fp8", "nvfp4")}


class KvBitsRefused(ValueError):
    """A request this engine cannot deploy; `fallback` (when set) is a plan that honours every ceiling asked for."""

    def __init__(self, message: str, fallback: Optional[BitBudgetPlan] = None, layer: Optional[int] = None):
        super().__init__(message)
        self.fallback, self.layer = fallback, layer


@dataclass
class ScoreTable:
    penalties: Dict[str, int]            # tier -> penalty x 1000
    provenance: str = "prior"            # "prior" = shipped needle-sweep priors; otherwise the file it was read from

    def apply(self, ladder: Dict[str, Tier]) -> Dict[str, Tier]:
        unknown = sorted(set(self.penalties) - set(ladder))
        if unknown:
            raise ValueError(f"score table names tiers the ladder does not have: {', '.join(unknown)}")
        return {n: replace(t, penalty_milli=self.penalties.get(n, t.penalty_milli)) for n, t in ladder.items()}


def default_scores(ladder: Optional[Dict[str, Tier]] = None) -> ScoreTable:
    ladder = ladder or build_ladder()
    return ScoreTable({n: t.penalty_milli for n, t in ladder.items()}, "prior")


def emit_scores(table: ScoreTable, ladder: Optional[Dict[str, Tier]] = None) -> str:
    ladder = ladder or build_ladder()
    lines = [f"# kv tier scores (penalty x 1000, lower is better); provenance: {table.provenance}",
             "# tier=penalty        bits/element"]
    for name, t in sorted(ladder.items(), key=lambda kv: -kv[1].bits_centi):
        lines.append(f"{name}={table.penalties.get(name, t.penalty_milli)}".ljust(22) + f"# {t.bits_centi / 100:.2f}")
    return "\n".join(lines) + "\n"


def parse_scores(text: str, provenance: str = "file") -> ScoreTable:
    out: Dict[str, int] = {}
    for ln, raw in enumerate(text.splitlines(), 1):
        line = raw.split("#", 1)[0].strip()
        if not line:
            continue
        name, sep, val = line.partition("=")
        if not sep or not name.strip() or not val.strip().lstrip("-").isdigit():
            raise ValueError(f"score table line {ln}: expected tier=penalty, got {raw!r}")
        if name.strip() in out:
            raise ValueError(f"score table line {ln}: tier {name.strip()!r} appears twice")
        out[name.strip()] = int(val)
    if not out:
        raise ValueError("score table is empty")
    return ScoreTable(out, provenance)


def _check_ceiling(bits: float, what: str, ladder: Dict[str, Tier]) -> None:
    if not MIN_BITS <= bits <= MAX_BITS:
        raise KvBitsRefused(f"{what} must lie in [{MIN_BITS}, {MAX_BITS}] bits per element, got {bits}")
    cheapest = min(ladder.values(), key=lambda t: t.bits_centi)
    if bits * 100 < cheapest.bits_centi:
        raise KvBitsRefused(f"{what} {bits} is below the cheapest tier the engine builds "
                            f"({cheapest.name}, {cheapest.bits_centi / 100:.2f} bits per element)")


def reachable_tiers(bits: float, ladder: Optional[Dict[str, Tier]] = None) -> List[str]:
    ladder = ladder or build_ladder()
    return [t.name for t in sorted(ladder.values(), key=lambda t: t.bits_centi) if t.bits_centi <= bits * 100 + 1e-9]


def entry_joint(n_layers: int, ceiling: float, scores: Optional[ScoreTable] = None,
                k_scores: Optional[ScoreTable] = None, v_scores: Optional[ScoreTable] = None) -> BitBudgetPlan:
    if k_scores is not None or v_scores is not None:
        raise KvBitsRefused("a per-plane score table has nothing to fit in the joint reading (one ceiling, one ladder): "
                            "give both ceilings, or pass the table as the common one")
    ladder = build_ladder()
    if scores is not None:
        ladder = scores.apply(ladder)
    _check_ceiling(ceiling, "the KV ceiling", ladder)
    return solve_bit_budget(n_layers, ceiling, ladder)


@dataclass
class SplitPlan:
    k_tiers: List[str]
    v_tiers: List[str]
    tiers: List[str]                 # the deployed tier per layer (the pair's builder)
    spec: str
    k_avg_bits: float
    v_avg_bits: float
    headroom_bits: Dict[str, float] = field(default_factory=dict)   # ceiling mode: what the wider plane could not spend


def _plane(n_layers: int, ceiling: float, table: Optional[ScoreTable], common: Optional[ScoreTable]) -> BitBudgetPlan:
    ladder = build_ladder()
    use = table or common                      # the common table is the fall-back of a plane without its own
    if use is not None:
        ladder = use.apply(ladder)
    return solve_bit_budget(n_layers, ceiling, ladder)


def entry_split(n_layers: int, k_ceiling: float, v_ceiling: float, scores: Optional[ScoreTable] = None,
                k_scores: Optional[ScoreTable] = None, v_scores: Optional[ScoreTable] = None,
                mode: str = "split") -> SplitPlan:
    if mode not in ("split", "ceiling"):
        raise KvBitsRefused(f"unknown K/V bits mode {mode!r} (split | ceiling)")
    ladder = build_ladder()
    _check_ceiling(k_ceiling, "the K ceiling", ladder)
    _check_ceiling(v_ceiling, "the V ceiling", ladder)
    if mode == "ceiling":
        low = min(k_ceiling, v_ceiling)
        plan = _plane(n_layers, low, None, scores)
        wide = "k" if k_ceiling > v_ceiling else "v"
        head = {wide: round(max(k_ceiling, v_ceiling) - plan.avg_bits, 4)} if k_ceiling != v_ceiling else {}
        return SplitPlan(list(plan.tiers), list(plan.tiers), list(plan.tiers), plan.spec, plan.avg_bits, plan.avg_bits, head)
    kp = _plane(n_layers, k_ceiling, k_scores, scores)
    vp = _plane(n_layers, v_ceiling, v_scores, scores)
    tiers: List[str] = []
    for i, (kt, vt) in enumerate(zip(kp.tiers, vp.tiers)):
        built = BUILDABLE_PAIRS.get((kt, vt))
        if built is None:
            fallback = _plane(n_layers, min(k_ceiling, v_ceiling), None, scores)
            raise KvBitsRefused(
                f"layer {i}: K wants {kt} and V wants {vt}, and no tier stores K as {kt} with V as {vt} (a layer's pages "
                f"carry one format for both planes).  Deployable instead, honouring both ceilings: the joint plan at "
                f"{min(k_ceiling, v_ceiling)} bits, '{fallback.spec}' ({fallback.avg_bits:.2f} bits per element); "
                f"--kv-bits-mode ceiling deploys it and reports the headroom", fallback, i)
        tiers.append(built)
    return SplitPlan(list(kp.tiers), list(vp.tiers), tiers, format_layer_storage(tiers), kp.avg_bits, vp.avg_bits)


def resolve(n_layers: int, bits: Optional[float] = None, k_bits: Optional[float] = None, v_bits: Optional[float] = None,
            mode: Optional[str] = None, scores: Optional[ScoreTable] = None, k_scores: Optional[ScoreTable] = None,
            v_scores: Optional[ScoreTable] = None):
    """The one resolution path of the front ends: which entry a set of flags means."""
    if k_bits is None and v_bits is None:
        if bits is None:
            raise KvBitsRefused("no KV ceiling given")
        if mode not in (None, "joint"):
            raise KvBitsRefused(f"--kv-bits-mode {mode} needs two ceilings (--kv-k-bits and --kv-v-bits); one ceiling has "
                                f"only the joint reading")
        return entry_joint(n_layers, bits, scores, k_scores, v_scores)
    if bits is not None:
        raise KvBitsRefused("give either one ceiling (--kv-bits) or the two per-plane ceilings, not both")
    if k_bits is None or v_bits is None:
        raise KvBitsRefused("the split reading needs both --kv-k-bits and --kv-v-bits")
    if mode == "joint":
        raise KvBitsRefused("--kv-bits-mode joint takes one ceiling (--kv-bits)")
    return entry_split(n_layers, k_bits, v_bits, scores, k_scores, v_scores, mode or "split")


def main(argv: Optional[Sequence[str]] = None) -> int:
    """`python -m ninfer_fusion_b200.kv.kv_bits score-table show|emit=<path>` and `plan` run without a model."""
    import argparse
    ap = argparse.ArgumentParser(prog="kv_bits")
    sub = ap.add_subparsers(dest="cmd", required=True)
    st = sub.add_parser("score-table", help="the ladder's penalty column: show it or write it as a loadable table")
    st.add_argument("action", help="show | emit=<path>")
    st.add_argument("--from", dest="src", default="", help="a score table file instead of the shipped priors")
    pl = sub.add_parser("plan", help="per-layer tiers for a ceiling (joint) or two ceilings (split / ceiling)")
    pl.add_argument("--layers", type=int, required=True)
    pl.add_argument("--kv-bits", type=float)
    pl.add_argument("--kv-k-bits", type=float)
    pl.add_argument("--kv-v-bits", type=float)
    pl.add_argument("--kv-bits-mode", default=None, choices=["joint", "split", "ceiling"])
    pl.add_argument("--kv-tier-scores", default="")
    pl.add_argument("--kv-k-tier-scores", default="")
    pl.add_argument("--kv-v-tier-scores", default="")
    a = ap.parse_args(argv)

    def load(path):
        if not path:
            return None
        with open(path) as f:
            return parse_scores(f.read(), path)
    if a.cmd == "score-table":
        table = load(a.src) or default_scores()
        text = emit_scores(table)
        if a.action == "show":
            print(text, end="")
            return 0
        if a.action.startswith("emit="):
            with open(a.action[5:], "w") as f:
                f.write(text)
            return 0
        ap.error("score-table takes show or emit=<path>")
    try:
        plan = resolve(a.layers, a.kv_bits, a.kv_k_bits, a.kv_v_bits, a.kv_bits_mode, load(a.kv_tier_scores),
                       load(a.kv_k_tier_scores), load(a.kv_v_tier_scores))
    except KvBitsRefused as e:
        print(f"refused: {e}")
        return 2
    print(plan.spec)
    print(plan)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
