"""Speculative-decoding options as the front ends spell them, and their validation.

One place turns the strings of the CLI, the server and the bench into a checked configuration, so that the three cannot
drift: backend names (`none` / `off`, `mtp`, `dflash`, `auto`; `dspark` names the DFlash runtime with the artifact's
Markov head and resolves to `dflash`), the draft width (MTP: 0 = adaptive over the width ladder, 1..15 pinned; DFlash:
1..15, the block width is fixed at start-up), the proposal head (`full`, `shortlist`, `auto` = shortlist when the
artifact carries one) and the draft tree shape `L,d` (L candidates per depth, d depths; 1 + L * d nodes must fit the
64-node verify window).  `resolve` then decides what `auto` means for the weights at hand.

Reference: src/product/speculative_options.h (backend spellings, width domains, which options need which backend).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional, Tuple

BACKENDS = ("none", "mtp", "dflash", "auto")
MAX_DRAFT_TOKENS = 15          # verify width cap of 16 rows per sequence
ADAPTIVE_MAX_WIDTH = 8         # widest rung captured when the width is left to the controller
MAX_TREE_NODES = 64            # one visibility bit per node of a verify window


def parse_backend(value: str) -> str:
    v = (value or "").strip().lower()
    if v in ("none", "off"):
        return "none"
    if v == "dspark":           # the Markov-head drafter IS the DFlash runtime; the artifact decides whether the head exists
        return "dflash"
    if v in BACKENDS:
        return v
    raise ValueError(f"invalid speculative backend: {value!r} (none | off | mtp | dflash | dspark | auto)")


def parse_tree(value: Optional[str]) -> Tuple[int, int]:
    """'L,d' -> (ranks per depth, depths); '' / None -> a chain (1, 0 = use the draft width)."""
    if not value:
        return 1, 0
    parts = value.split(",")
    if len(parts) != 2 or not all(p.strip().isdigit() for p in parts):
        raise ValueError(f"--draft-tree takes L,d (two positive integers), got {value!r}")
    ranks, depths = int(parts[0]), int(parts[1])
    if ranks < 1 or depths < 1:
        raise ValueError("--draft-tree: L and d must be at least 1")
    if 1 + ranks * depths > MAX_TREE_NODES:
        raise ValueError(f"--draft-tree {value}: {1 + ranks * depths} nodes exceed the {MAX_TREE_NODES}-node verify window")
    return ranks, depths


@dataclass(frozen=True)
class SpeculativeOptions:
    backend: str = "none"
    draft_tokens: int = 0              # 0: MTP adaptive / backend default
    proposal_head: str = "auto"        # full | shortlist | auto
    tree_ranks: int = 1
    tree_depths: int = 0
    stochastic_drafts: bool = False

    def validate(self) -> "SpeculativeOptions":
        if self.backend not in BACKENDS:
            raise ValueError(f"invalid speculative backend: {self.backend!r}")
        if self.proposal_head not in ("full", "shortlist", "auto"):
            raise ValueError(f"invalid proposal head: {self.proposal_head!r} (full | shortlist | auto)")
        if self.draft_tokens < 0:
            raise ValueError("--draft-tokens must not be negative")
        tree = self.tree_ranks > 1
        if self.backend in ("none", "auto"):
            # auto's whole job is to resolve the backend; pinning a width or a head is spelled with an explicit one
            if self.draft_tokens != 0 or self.proposal_head == "shortlist" or tree or self.stochastic_drafts:
                raise ValueError("--draft-tokens, --draft-head, --draft-tree and --spec-stochastic require --spec mtp|dflash")
            return self
        if self.backend == "mtp":
            if self.draft_tokens > MAX_DRAFT_TOKENS:
                raise ValueError(f"--spec mtp requires --draft-tokens in [0,{MAX_DRAFT_TOKENS}] (0 = adaptive)")
            if tree and self.draft_tokens == 0:
                raise ValueError("a draft tree has a fixed shape: give its depth with --draft-tree L,d")
            if tree and (self.proposal_head == "shortlist" or self.stochastic_drafts):
                raise ValueError("a draft tree ranks candidates over the full distribution: no shortlist head, no sampled drafts")
            if self.stochastic_drafts and self.proposal_head == "shortlist":
                raise ValueError("sampled drafts export their distribution over the full vocabulary: no shortlist head")
            return self
        # dflash
        if not 1 <= self.draft_tokens <= MAX_DRAFT_TOKENS:
            raise ValueError(f"--spec dflash requires --draft-tokens in [1,{MAX_DRAFT_TOKENS}]")
        if tree or self.stochastic_drafts:
            raise ValueError("the DFlash drafter proposes one arg-max chain per round")
        return self

    def resolve(self, has_draft_module: bool, has_dflash: bool, has_shortlist: bool) -> "SpeculativeOptions":
        """What runs for the weights at hand: `auto` picks the draft module when the artifact has one, an explicit
        backend whose weights are missing is refused, `auto` head means the shortlist when there is one."""
        o = self.validate()
        if o.backend == "auto":
            o = replace(o, backend="mtp" if has_draft_module else "none")
        if o.backend == "mtp" and not has_draft_module:
            raise ValueError("--spec mtp: the weights have no draft module")
        if o.backend == "dflash" and not has_dflash:
            raise ValueError("--spec dflash: the weights have no DFlash draft model")
        if o.backend == "none":
            return replace(o, proposal_head="full")
        head = o.proposal_head
        if head == "shortlist" and not has_shortlist:
            raise ValueError("the artifact carries no shortlist draft head (text/draft_head_token_ids)")
        if head == "auto":
            head = "shortlist" if has_shortlist and o.tree_ranks == 1 and not o.stochastic_drafts else "full"
        return replace(o, proposal_head=head)

    @property
    def adaptive(self) -> bool:
        return self.backend == "mtp" and self.draft_tokens == 0 and self.tree_ranks == 1

    @property
    def width(self) -> int:
        """Drafts per round the buffers are sized for."""
        if self.tree_ranks > 1:
            return self.tree_depths
        return self.draft_tokens or (ADAPTIVE_MAX_WIDTH if self.backend == "mtp" else 0)


def from_strings(spec: str = "none", draft_tokens: int = 0, proposal_head: str = "auto", draft_tree: Optional[str] = None,
                 stochastic: bool = False) -> SpeculativeOptions:
    ranks, depths = parse_tree(draft_tree)
    return SpeculativeOptions(parse_backend(spec), int(draft_tokens), proposal_head, ranks, depths, bool(stochastic)).validate()
