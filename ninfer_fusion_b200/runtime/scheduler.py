"""Scheduling decisions of the engine worker, kept apart from the worker loop so that they can be tested as functions.

* **Execution choice.**  One unit of work per iteration: a prefill unit or a decode round.  With both kinds runnable
  the two alternate 1:1; the bandwidth governor's verdict can hold prefill back while decode work exists; with no
  decode lanes prefill always runs (prefill cannot starve).
* **Service quanta.**  A request's remaining work is counted in quanta: one per prefill unit still to run and one per
  token still to generate.  The number of prefill quanta depends on the unit in force, so when the governor shrinks
  the unit mid-prompt the not-yet-charged span is re-priced (monotone: growing the unit back never refunds).
* **Blocked FIFO head and back-fill.**  Admission is FIFO.  When the head does not fit, the requests that are active
  at that moment are frozen as its *donors*: the head becomes runnable when they leave.  A request behind the head may
  be admitted out of order (a *borrower*) only with a proof from the Program that the head still fits once every donor
  has left and the borrower is still resident; borrowers never become donors of the same protection, so repeated
  back-fill cannot push the head's turn away; with no live donor left nothing is back-filled (the head is waiting for
  borrowers, and more of them would starve it).

Reference: src/runtime/engine/scheduler.h (choose_execution :291-300, service-work accounting :236-283, FIFO snapshot
with back-fill candidates), src/runtime/engine/admission_policy.h (protection epochs, donors, persistent back-fill).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import FrozenSet, Iterable, Optional, Set


class ExecutionAction(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    WAIT = "wait"


def choose_execution(have_decode: bool, prefill_runnable: bool, previous_unit_was_decode: bool,
                     prefill_admitted: bool = True) -> ExecutionAction:
    if prefill_runnable:
        if have_decode and (not previous_unit_was_decode or not prefill_admitted):
            return ExecutionAction.DECODE
        return ExecutionAction.PREFILL
    return ExecutionAction.DECODE if have_decode else ExecutionAction.WAIT


def prefill_quanta_for(tokens: int, unit: int) -> int:
    """Prefill units a span of `tokens` needs at `unit` tokens per unit."""
    return 0 if tokens <= 0 or unit <= 0 else 1 + (tokens - 1) // unit


def projected_service_work(prompt_tokens_left: int, unit: int, max_new_tokens: int) -> int:
    return prefill_quanta_for(prompt_tokens_left, unit) + max(0, int(max_new_tokens))


@dataclass
class ServiceAccount:
    """Remaining service work of one request, in quanta."""
    remaining: int
    unit: int                      # prefill unit the reservation was last reconciled against

    def consume(self, work: int = 1) -> None:
        if work <= 0 or work > self.remaining:
            raise RuntimeError(f"request service projection consumed {work} quanta with {self.remaining} remaining")
        self.remaining -= work

    def reconcile(self, prompt_tokens_left: int, unit: int) -> None:
        """The prefill unit moved: re-price the span that has not been charged yet.  Only ever adds."""
        before = prefill_quanta_for(prompt_tokens_left, self.unit)
        after = prefill_quanta_for(prompt_tokens_left, unit)
        if after > before:
            self.remaining += after - before
        self.unit = unit


@dataclass
class AdmissionProtection:
    epoch: int
    head_id: int
    donors: FrozenSet[int]
    borrowers: Set[int] = field(default_factory=set)

    def live_donors(self, active: Iterable[int]) -> FrozenSet[int]:
        return self.donors & frozenset(active)


class Scheduler:
    def __init__(self) -> None:
        self.previous_unit_was_decode = True    # so that the first runnable prefill unit is not held behind a round
        self.protection: Optional[AdmissionProtection] = None
        self._epoch = 0
        self.stats = {"protections": 0, "backfills": 0, "backfill_refusals": 0, "prefill_holds": 0}

    # ------------------------------------------------------------------ execution
    def choose(self, have_decode: bool, prefill_runnable: bool, prefill_admitted: bool = True) -> ExecutionAction:
        action = choose_execution(have_decode, prefill_runnable, self.previous_unit_was_decode, prefill_admitted)
        if prefill_runnable and have_decode and not prefill_admitted and action is ExecutionAction.DECODE \
                and self.previous_unit_was_decode:
            self.stats["prefill_holds"] += 1
        return action

    def ran(self, action: ExecutionAction) -> None:
        if action is not ExecutionAction.WAIT:
            self.previous_unit_was_decode = action is ExecutionAction.DECODE

    # ------------------------------------------------------------------ blocked head
    def observe_head(self, head_id: Optional[int]) -> None:
        """A protection belongs to one head: it ends when that request is admitted, cancelled or times out."""
        if self.protection is not None and self.protection.head_id != head_id:
            self.protection = None

    def protect(self, head_id: int, active: Iterable[int]) -> AdmissionProtection:
        """The head does not fit: freeze who it is waiting for (once per head)."""
        if self.protection is None or self.protection.head_id != head_id:
            self._epoch += 1
            self.protection = AdmissionProtection(self._epoch, head_id, frozenset(active))
            self.stats["protections"] += 1
        return self.protection

    def authorize_backfill(self, candidate_id: int, active: Iterable[int], proof: bool) -> bool:
        """May `candidate_id` overtake the blocked head?  `proof` is the Program's statement that the head still
        fits after every live donor has left with the candidate resident."""
        p = self.protection
        ok = p is not None and candidate_id != p.head_id and bool(p.live_donors(active)) and bool(proof)
        if ok:
            p.borrowers.add(candidate_id)
            self.stats["backfills"] += 1
        else:
            self.stats["backfill_refusals"] += 1
        return ok
