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
