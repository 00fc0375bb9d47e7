"""Per-cell KV precision descent.

A *cell* is one page-sized block of tokens in one full-attention layer.  Every cell sits on a rung
of a tier ladder (highest precision first).  A descent pass lowers selected cells by exactly ONE
rung, oldest blocks first, under three budgets (cells per pass, bytes freed per pass, resident-byte
target) and an age gate that protects the most recent tokens; a cell that already sits on the
last rung is a candidate for the cold tier instead.  This mirrors the reference's block-descent
planner contract (src/product/kv_block_descent.h:1-58: one rung per pass, rate / bytes / blocks
budgets, age gate, carry re-anchoring) as a host-only function: the engine applies the returned moves
with the requantise kernel and publishes the new block-table tags.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .policy import Tier, build_ladder


@dataclass(frozen=True)
class DescentConfig:
    ladder: Tuple[str, ...] = ("bf16", "fp8", "nvfp4")   # rungs, highest precision first
    min_age_tokens: int = 2048        # blocks whose last token is younger than this stay untouched
    max_cells_per_pass: int = 256
    max_bytes_per_pass: int = 1 << 30
    target_resident_bytes: int = 0    # 0 = no target: descend whatever the other budgets allow
    sink_blocks: int = 1              # leading blocks of a sequence that never descend (attention sinks)
    floor: str = ""                   # ladder tier below which no cell descends ("" = the ladder's last rung)
    # stateless solve instead of the incremental walk: with a cost table (and a resident-bytes target) every pass solves
    # the whole allocation afresh and moves cells one rung toward it; a refusal moves nothing
    solve_table: Optional["CellCostTable"] = None


@dataclass(frozen=True)
class Move:
    seq: int
    layer: int
    block: int
    src: str
    dst: str          # a ladder tier, or "cold"
    bytes_freed: int


@dataclass
class CellMap:
    """Rung index of every (sequence, layer, block) cell; `frontier[seq]` = tokens written so far."""
    page_tokens: int
    n_layers: int
    rungs: Dict[Tuple[int, int, int], int] = field(default_factory=dict)
    frontier: Dict[int, int] = field(default_factory=dict)

    def touch(self, seq: int, n_tokens: int) -> None:
        """Register blocks up to the frontier at rung 0 (new KV is always written at full precision)."""
        self.frontier[seq] = n_tokens
        n_blocks = (n_tokens + self.page_tokens - 1) // self.page_tokens
        for layer in range(self.n_layers):
            for b in range(n_blocks):
                self.rungs.setdefault((seq, layer, b), 0)

    def drop(self, seq: int) -> None:
        self.frontier.pop(seq, None)
        for k in [k for k in self.rungs if k[0] == seq]:
            del self.rungs[k]

    def trim(self, seq: int, n_tokens: int) -> None:
        """Speculative rollback: forget cells wholly beyond the new frontier."""
        keep = (n_tokens + self.page_tokens - 1) // self.page_tokens
        for k in [k for k in self.rungs if k[0] == seq and k[2] >= keep]:
            del self.rungs[k]
        self.frontier[seq] = n_tokens


def cell_bytes(tier: Tier, page_tokens: int, n_kv_heads: int, head_dim: int) -> int:
    return 2 * page_tokens * n_kv_heads * head_dim * tier.bits_centi // 800


def resident_bytes(cells: CellMap, cfg: DescentConfig, tiers: Dict[str, Tier], n_kv_heads: int, head_dim: int) -> int:
    per = [cell_bytes(tiers[name], cells.page_tokens, n_kv_heads, head_dim) for name in cfg.ladder]
    return sum(per[r] for r in cells.rungs.values() if r < len(per))


def plan_descent_pass(cells: CellMap, cfg: DescentConfig, n_kv_heads: int, head_dim: int,
                      tiers: Optional[Dict[str, Tier]] = None, allow_cold: bool = False) -> List[Move]:
    """One pass: at most one rung per cell, oldest first (ties: shallow layer first, then sequence id)."""
    tiers = tiers or build_ladder(head_dim)
    if cfg.solve_table is not None and cfg.target_resident_bytes > 0 and not allow_cold:
        alloc = solve_cell_allocation(cells, cfg, cfg.target_resident_bytes, cfg.solve_table, n_kv_heads, head_dim, tiers)
        return moves_toward(cells, cfg, alloc, n_kv_heads, head_dim, tiers) if alloc.outcome == SOLVED else []
    per = [cell_bytes(tiers[name], cells.page_tokens, n_kv_heads, head_dim) for name in cfg.ladder]
    last = len(cfg.ladder) - 1
    if cfg.floor:
        if cfg.floor not in cfg.ladder:
            raise ValueError(f"descent floor '{cfg.floor}' is not a rung of the ladder {cfg.ladder}")
        last = cfg.ladder.index(cfg.floor)     # the `cold=` tier of the tier-format grammar: the deepest resident rung
    resident = resident_bytes(cells, cfg, tiers, n_kv_heads, head_dim)
    cands = []
    for (seq, layer, block), rung in cells.rungs.items():
        if block < cfg.sink_blocks:
            continue
        age = cells.frontier.get(seq, 0) - (block + 1) * cells.page_tokens
        if age < cfg.min_age_tokens:
            continue
        if rung < last:
            cands.append((-age, layer, seq, block, rung))
        elif rung == last and allow_cold:
            cands.append((-age, layer, seq, block, rung))
    cands.sort()
    moves: List[Move] = []
    freed = 0
    for _, layer, seq, block, rung in cands:
        if len(moves) >= cfg.max_cells_per_pass:
            break
        if cfg.target_resident_bytes and resident - freed <= cfg.target_resident_bytes:
            break
        if rung < last:
            gain = per[rung] - per[rung + 1]
            dst = cfg.ladder[rung + 1]
        else:
            gain = per[rung]
            dst = "cold"
        if freed + gain > cfg.max_bytes_per_pass and moves:
            break
        moves.append(Move(seq, layer, block, cfg.ladder[rung], dst, gain))
        freed += gain
    return moves


def apply_moves(cells: CellMap, cfg: DescentConfig, moves: Sequence[Move]) -> None:
    for m in moves:
        key = (m.seq, m.layer, m.block)
        cells.rungs[key] = len(cfg.ladder) if m.dst == "cold" else cfg.ladder.index(m.dst)


# ----------------------------------------------------------------------------- the stateless allocation solve
# The walk above moves one rung per cell and pass because it MODIFIES what the next pass sees and needs a reason to
# stop.  A solve computes the whole allocation from its inputs in one go, so it may take a cell down any number of rungs
# at once and carries nothing between passes: it is re-solved from the measurement every time, which is the shape that
# survives a churning population of cells.  Its only quality constraint is ONE measured precision floor (the total loss,
# in nats, the allocation may spend); a budget that cannot be reached inside that floor is refused BY NAME and the
# status quo is returned: a silent compromise would leave the precision undetermined.
# Reference: src/product/kv_cell_alloc_solve.h (stateless solve, floor as the one constraint, named refusals, one-way
# prefix family per cell, oldest-first tie-break, position-blind rule).
@dataclass(frozen=True)
class CellCostTable:
    rung_cost_nats: Tuple[float, ...]   # loss of taking one cell INTO rung i (index 0 unused: nothing descends into it)
    floor_nats: float                   # total loss the allocation may spend
    floor_measured: bool = False        # a prior is not a measurement: an unmeasured floor is refused unless allowed


SOLVED, NO_PRESSURE = "solved", "no_pressure"
REFUSED_FLOOR_UNMEASURED = "refused_floor_unmeasured"
REFUSED_BUDGET_UNREACHABLE = "refused_budget_unreachable_within_floor"
REFUSED_EMPTY, REFUSED_BAD_TABLE = "refused_no_cells", "refused_bad_cost_table"


@dataclass
class CellAllocation:
    outcome: str
    target: Dict[Tuple[int, int, int], int]     # rung of every cell in the solved allocation (status quo on a refusal)
    resident_bytes: int
    budget_bytes: int
    spent_nats: float = 0.0
    cells_demoted: int = 0
    deficit_bytes: int = 0                      # on the budget refusal: what is still missing at the floor


def solve_cell_allocation(cells: CellMap, cfg: DescentConfig, budget_bytes: int, table: CellCostTable,
                          n_kv_heads: int, head_dim: int, tiers: Optional[Dict[str, Tier]] = None,
                          allow_unmeasured_floor: bool = False) -> CellAllocation:
    import heapq
    tiers = tiers or build_ladder(head_dim)
    per = [cell_bytes(tiers[name], cells.page_tokens, n_kv_heads, head_dim) for name in cfg.ladder]
    status_quo = dict(cells.rungs)
    resident = sum(per[r] for r in status_quo.values() if r < len(per))
    if not status_quo:
        return CellAllocation(REFUSED_EMPTY, status_quo, 0, budget_bytes)
    if len(table.rung_cost_nats) != len(cfg.ladder) or any(c < 0 for c in table.rung_cost_nats) or table.floor_nats < 0:
        return CellAllocation(REFUSED_BAD_TABLE, status_quo, resident, budget_bytes)
    if resident <= budget_bytes:
        return CellAllocation(NO_PRESSURE, status_quo, resident, budget_bytes)
    if not table.floor_measured and not allow_unmeasured_floor:
        return CellAllocation(REFUSED_FLOOR_UNMEASURED, status_quo, resident, budget_bytes)
    last = cfg.ladder.index(cfg.floor) if cfg.floor else len(cfg.ladder) - 1

    def step(key, rung):
        """The next step of a cell's own chain as a heap entry: cheapest loss per byte first; among equals the oldest
        block, then the shallower layer, then the sequence id.  Nothing here reads a position inside a block."""
        gain = per[rung] - per[rung + 1]
        cost = table.rung_cost_nats[rung + 1]
        return (cost / gain if gain > 0 else float("inf"), key[2], key[1], key[0], rung)
    heap = []
    for key, rung in status_quo.items():
        seq, layer, block = key
        if block < cfg.sink_blocks or rung >= last:
            continue
        if cells.frontier.get(seq, 0) - (block + 1) * cells.page_tokens < cfg.min_age_tokens:
            continue
        heapq.heappush(heap, step(key, rung))
    target = dict(status_quo)
    spent = 0.0
    while resident > budget_bytes and heap:
        ratio, block, layer, seq, rung = heapq.heappop(heap)
        key = (seq, layer, block)
        if target[key] != rung:          # prefix guard: a cell walks its own chain in order, one way only
            continue
        cost = table.rung_cost_nats[rung + 1]
        if spent + cost > table.floor_nats + 1e-12:
            continue                     # this step would cross the floor; a cheaper-in-nats step may still fit
        spent += cost
        resident -= per[rung] - per[rung + 1]
        target[key] = rung + 1
        if rung + 1 < last:
            heapq.heappush(heap, step(key, rung + 1))
    if resident > budget_bytes:
        start = sum(per[r] for r in status_quo.values() if r < len(per))
        return CellAllocation(REFUSED_BUDGET_UNREACHABLE, status_quo, start, budget_bytes, 0.0, 0, resident - budget_bytes)
    demoted = sum(1 for k, r in target.items() if r != status_quo[k])
    return CellAllocation(SOLVED, target, resident, budget_bytes, spent, demoted)


def moves_toward(cells: CellMap, cfg: DescentConfig, alloc: CellAllocation, n_kv_heads: int, head_dim: int,
                 tiers: Optional[Dict[str, Tier]] = None) -> List[Move]:
    """One pass of device work toward a solved allocation: every cell that is above its target moves ONE rung (the
    re-encoding kernel goes rung by rung), oldest first, under the pass budgets.  Re-solving next pass needs no memory
    of this one."""
    tiers = tiers or build_ladder(head_dim)
    per = [cell_bytes(tiers[name], cells.page_tokens, n_kv_heads, head_dim) for name in cfg.ladder]
    due = sorted((k[2], k[1], k[0]) for k, r in cells.rungs.items() if alloc.target.get(k, r) > r)
    moves: List[Move] = []
    freed = 0
    for block, layer, seq in due:
        r = cells.rungs[(seq, layer, block)]
        gain = per[r] - per[r + 1]
        if len(moves) >= cfg.max_cells_per_pass or (freed + gain > cfg.max_bytes_per_pass and moves):
            break
        moves.append(Move(seq, layer, block, cfg.ladder[r], cfg.ladder[r + 1], gain))
        freed += gain
    return moves

