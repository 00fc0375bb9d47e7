"""History look-up drafts: which tokens of a draft block the sequence's own history can fill, and when that copy
signal has earned the wide verify round.

* `suffix_best`: the newest Q tokens of a sequence are the query; find the longest earlier occurrence of the query's
  tail (match length L <= Q, at least `min_len`; ties prefer the LATEST occurrence).  A candidate window must lie
  strictly before the query and leave the whole K-token continuation inside the history: an overlapping window's
  "continuation" is the query itself, which is not new information.  One function states that bound
  (`scan_limit`), everything else asks it.
* `fuse_chain`: the draft policy.  Full match (L == Q): propose K tokens straight from the history (the drafter does
  not take part).  Partial match (min_len <= L < Q): propose ONE probe token, the history's token after the matched
  part; the next round's query then contains it and the match can grow.  Below `min_len`: nothing, the neural
  drafter proposes.  The history position every proposed token was copied from is returned too (a retention policy
  keyed on which pages drafts come from needs it; page = position // page_tokens).
* `VerifyWidthController`: two rungs, narrow (the neural block) and wide (narrow + slots only the history can fill).
  The wide rung is earned by ONE request over ITS consecutive strong-copy rounds, needs the look-up to fill EVERY
  extra slot (a short continuation is a refusal, never a narrower wide round), falls back on the first miss, may
  coast through at most `coast_rounds` weak rounds when a single request is decoding, and is never sticky across
  requests.

Reference: src/spec/lookup_fuse.h (chain policy, copied-from positions), include/ninfer/ops/suffix_lookup.h (match
definition, scan bound), src/spec/labd_verify_width.h (the width decision as a state machine over integers).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple


def scan_limit(start: int, length: int, query: int, continuation_tokens: int) -> int:
    """Candidate offsets o in [0, scan_limit): strictly earlier (o + Q < start) with room for the continuation."""
    return min(length - query - continuation_tokens, start - query)


def suffix_best(ids: Sequence[int], query_start: int, query_len: int, min_len: int,
                continuation_tokens: int = 0) -> Tuple[int, int]:
    """(match length, window offset) of the best earlier occurrence of the query's tail; (0, 0) when none."""
    best_len, best_off = 0, 0
    q_end = query_start + query_len
    for o in range(max(0, scan_limit(query_start, len(ids), query_len, continuation_tokens))):
        l = 0
        while l < query_len and ids[q_end - 1 - l] == ids[o + query_len - 1 - l]:
            l += 1
        if l >= min_len and (l > best_len or (l == best_len and o > best_off)):
            best_len, best_off = l, o
    return best_len, best_off


def fuse_chain(ids: Sequence[int], query_len: int, min_len: int, k: int,
               query_start: Optional[int] = None) -> Tuple[List[int], List[int], int]:
    """(proposed tokens, the history positions they were copied from, match length).  Empty lists: fall back."""
    n = len(ids)
    query_len = min(query_len, n)
    if query_len < 1 or k < 1:
        return [], [], 0
    start = n - query_len if query_start is None else query_start
    length, off = suffix_best(ids, start, query_len, min_len, k)
    if length < min_len:
        return [], [], length
    want = k if length == query_len else 1
    toks, src = [], []
    for j in range(want):
        pos = off + query_len + j
        if pos >= n:
            break
        toks.append(int(ids[pos]))
        src.append(pos)
    return toks, src, length


def lookup_drafter(history: Sequence[int], k: int, query_len: int = 8, min_len: int = 2) -> Optional[List[int]]:
    """The chain policy as a drafter hook: K draft tokens or None.  A one-token probe is padded by walking on through
    the history after it (the padding is only a guess; the verifier decides)."""
    toks, src, _ = fuse_chain(history, query_len, min_len, k)
    if not toks:
        return None
    pos = src[-1] + 1
    while len(toks) < k:
        toks.append(int(history[pos]) if pos < len(history) else toks[-1])
        pos += 1
    return toks


@dataclass
class VerifyWidthController:
    narrow: int = 8                 # columns of the narrow round: anchor + neural drafts
    wide: int = 16                  # columns of the wide round: narrow + look-up slots
    promote_after: int = 2          # consecutive strong rounds of one request before the wide rung
    coast_rounds: int = 3           # weak rounds a lone request may stay wide
    strong_len: int = 8             # a match at least this long is a strong copy signal
    width: int = field(init=False)
    _owner: Optional[int] = field(default=None, init=False)
    _streak: int = field(default=0, init=False)
    _coast: int = field(default=0, init=False)
    refusals: dict = field(default_factory=lambda: {"short_continuation": 0, "other_request": 0, "miss": 0})

    def __post_init__(self) -> None:
        if not 1 < self.narrow < self.wide:
            raise ValueError("the wide rung must be wider than the narrow one")
        self.width = self.narrow

    @property
    def lookup_slots(self) -> int:
        return self.wide - self.narrow

    def observe(self, request_id: int, requests: int, match_len: int, continuation: int, accepted_all: bool = True) -> int:
        """One round of `request_id` among `requests` concurrent ones: its look-up matched `match_len` tokens and can
        supply `continuation` tokens; `accepted_all` = the verifier took every look-up token of the last wide round.
        Returns the width of the NEXT round."""
        strong = match_len >= self.strong_len and accepted_all
        if self._owner is not None and request_id != self._owner:
            # a latch belongs to the request that earned it
            self.refusals["other_request"] += 1
            self._owner, self._streak, self._coast, self.width = request_id, 0, 0, self.narrow
        self._owner = request_id
        if strong:
            self._streak += 1
            self._coast = 0
            if continuation < self.lookup_slots:
                # the extra columns exist only because history tokens occupy them: all of them, or no wide round
                self.refusals["short_continuation"] += 1
                self.width = self.narrow
            elif self._streak >= self.promote_after:
                self.width = self.wide
            return self.width
        self._streak = 0
        if self.width == self.wide and requests == 1 and match_len > 0 and self._coast < self.coast_rounds:
            self._coast += 1            # a lone request may coast through a weak round or two
            return self.width
        if self.width == self.wide:
            self.refusals["miss"] += 1
        self.width, self._coast = self.narrow, 0
        return self.width
