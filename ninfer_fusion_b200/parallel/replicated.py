"""Multi-rank engine: one leader decides, every rank executes the same Program step.

A tensor- or expert-parallel model lives on W ranks (one process per GPU), but
there is one HTTP / CLI front end and one `Engine`.  The leader (rank 0) wraps
its shard's Program in `LeaderProgram`; every verb the engine calls on it is
first broadcast to the followers as one packed step descriptor, then executed
locally, so that all ranks walk through identical lane tables, page tables and
kernel launches (the peer-memory kernels of `parallel.tp` need every rank in
the same step).  Followers run `follower_loop` around their own shard.

Resource verdicts are AND-reduced: a request is admitted only if EVERY rank
can admit it, and a lane that one rank failed to open is closed again on all
ranks (the reference states both rules for its replicated residency decisions:
docs/maintainer/multi-device-and-shard-plan.md:111-160, the 2-rank AND of the
admit verdict in src/core/and_reduce.h:392-412; its world / rank environment
contract NINFER_WORLD_SIZE / NINFER_RANK is src/core/shard_plan.h:707-708).

Failure domains: an exception a follower raises while opening a lane fails
that request on every rank (request domain); a rank that stops answering makes
the next collective of the control channel time out, which the leader turns
into an engine-wide `ResourceError` (the engine then refuses work until
`recover()` builds a new Program, with a new channel, from its factory).

The control channel is a `torch.distributed` group on the `gloo` backend (host
memory only: it must keep working while the GPUs are busy, and it must fail by
time-out rather than hang).  Hot verbs (prefill step, decode round, close,
checkpoint) travel as one fixed-size int64 tensor; only `open` ships Python
objects (the prompt and its sampling parameters).
"""
from __future__ import annotations

import datetime
import os
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..runtime.engine import RequestError, ResourceError

OP_STOP, OP_CAN_ADMIT, OP_OPEN, OP_CLOSE, OP_PREFILL, OP_DECODE, OP_CHECKPOINT, OP_PING, OP_DESCENT, OP_FORCE = range(10)
_DESC_WORDS = 72   # op, count, then up to 64 lane ids / scalar arguments
_KINDS = ("turn", "endpoint", "replay", "anchor", "shared")


def world_from_env() -> tuple[int, int]:
    """(rank, world) from the launcher's environment: torchrun's RANK / WORLD_SIZE, else the reference's
    NINFER_RANK / NINFER_WORLD_SIZE, else a single rank."""
    for r, w in (("RANK", "WORLD_SIZE"), ("NINFER_RANK", "NINFER_WORLD_SIZE")):
        if w in os.environ:
            return int(os.environ.get(r, "0")), int(os.environ[w])
    return 0, 1


class RankChannel:
    """Control channel between the ranks of one engine (gloo group, bounded waits)."""

    def __init__(self, group, rank: int, world: int):
        self.group, self.rank, self.world = group, rank, world
        self._desc = torch.zeros(_DESC_WORDS, dtype=torch.int64)

    @classmethod
    def create(cls, rank: int, world: int, timeout_s: float = 30.0, ranks: Optional[Sequence[int]] = None) -> "RankChannel":
        """A gloo subgroup of the initialised default process group (all ranks must call this together)."""
        group = dist.new_group(ranks=list(ranks) if ranks is not None else None, backend="gloo",
                               timeout=datetime.timedelta(seconds=timeout_s))
        return cls(group, rank, world)

    # --- leader -> all ---
    def send_desc(self, op: int, args: Sequence[int] = ()) -> None:
        if len(args) > _DESC_WORDS - 2:
            raise ValueError("step descriptor overflow")
        d = self._desc
        d.zero_()
        d[0], d[1] = op, len(args)
        if args:
            d[2:2 + len(args)] = torch.tensor(list(args), dtype=torch.int64)
        self._collective(lambda: dist.broadcast(d, src=self._src(), group=self.group))

    def recv_desc(self) -> tuple[int, List[int]]:
        d = self._desc
        self._collective(lambda: dist.broadcast(d, src=self._src(), group=self.group))
        n = int(d[1])
        return int(d[0]), d[2:2 + n].tolist()

    def bcast_object(self, obj=None):
        box = [obj]
        self._collective(lambda: dist.broadcast_object_list(box, src=self._src(), group=self.group))
        return box[0]

    # --- verdicts ---
    def and_reduce(self, ok: bool) -> bool:
        """True iff every rank said True."""
        t = torch.tensor([1 if ok else 0], dtype=torch.int32)
        self._collective(lambda: dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group))
        return bool(int(t[0]))

    def gather_errors(self, err: Optional[str]) -> List[Optional[str]]:
        out: List[Optional[str]] = [None] * self.world
        self._collective(lambda: dist.all_gather_object(out, err, group=self.group))
        return out

    def _src(self) -> int:
        return dist.get_global_rank(self.group, 0) if self.group is not None else 0

    def _collective(self, fn: Callable[[], None]) -> None:
        try:
            fn()
        except Exception as e:  # noqa: BLE001 - time-out, closed connection, aborted peer: all the same verdict
            raise ResourceError(f"rank channel failed on rank {self.rank} ({type(e).__name__}: {e}): "
                                "a rank of this engine stopped answering") from e


def _sampling_to_wire(sp):
    return None if sp is None else dict(vars(sp))


def _sampling_from_wire(d):
    from ..runtime.program import SamplingParams
    return None if d is None else SamplingParams(**d)


class LeaderProgram:
    """Rank 0's view of the replicated Program: same verbs, every one mirrored on the followers first."""

    def __init__(self, inner, channel: RankChannel):
        self.inner, self.ch = inner, channel
        self.replicated_stats = {"steps": 0, "admit_vetoes": 0, "open_failures": 0}

    # read-only surface the engine and the service look at
    def __getattr__(self, name):
        return getattr(self.inner, name)

    def free_lanes(self) -> int:
        return self.inner.free_lanes()

    def census(self) -> dict:
        c = self.inner.census()
        c["ranks"] = self.ch.world
        c["replicated"] = dict(self.replicated_stats)
        return c

    # ---- verbs ----
    def can_admit(self, n_prompt: int, max_new: int) -> bool:
        self.ch.send_desc(OP_CAN_ADMIT, (n_prompt, max_new))
        mine = self.inner.can_admit(n_prompt, max_new)
        ok = self.ch.and_reduce(mine)
        if mine and not ok:
            self.replicated_stats["admit_vetoes"] += 1
        return ok

    def open(self, prompt, sampling=None, session=None, media=None):
        if media is not None:
            raise RequestError("media prompts are not supported by the multi-rank engine")
        self.ch.send_desc(OP_OPEN)
        # the lane id travels with the request: ids stay equal on all ranks even after an open that only some
        # ranks completed
        self.ch.bcast_object((list(prompt), _sampling_to_wire(sampling), session, int(self.inner._next_id)))
        lane, err = _try_open(self.inner, prompt, sampling, session)
        errs = self.ch.gather_errors(err)
        bad = [(r, e) for r, e in enumerate(errs) if e is not None]
        if bad:
            if lane is not None:
                self.inner.close(lane)   # every rank that did open the lane closes it again (followers do the same)
            self.replicated_stats["open_failures"] += 1
            r, e = bad[0]
            kind, _, text = e.partition(":")
            exc = RequestError if all(b[1].startswith("request:") for b in bad) else ResourceError
            raise exc(f"rank {r} could not open the lane: {text}")
        return lane

    def close(self, lane) -> None:
        self.ch.send_desc(OP_CLOSE, (lane.lane_id,))
        self.inner.close(lane)

    def prefill_step(self, lane, budget: int):
        self.ch.send_desc(OP_PREFILL, (lane.lane_id, int(budget)))
        self.replicated_stats["steps"] += 1
        return self.inner.prefill_step(lane, budget)

    def decode_round(self, lanes):
        ids = [l.lane_id for l in lanes]
        self.ch.send_desc(OP_DECODE, ids)
        self.replicated_stats["steps"] += 1
        return self.inner.decode_round(lanes)

    def force_next_token(self, lane, token: int) -> None:
        self.ch.send_desc(OP_FORCE, (lane.lane_id, int(token)))
        self.inner.force_next_token(lane, token)

    def checkpoint(self, lane, session, kind: str) -> bool:
        self.ch.send_desc(OP_CHECKPOINT, (lane.lane_id, _KINDS.index(kind)))
        self.ch.bcast_object(session)
        return self.inner.checkpoint(lane, session, kind)

    def kv_descent_step(self) -> int:
        """Per-cell KV precision descent, on every rank in the same step (each rank re-encodes its own heads)."""
        if getattr(self.inner, "descent", None) is None:
            return 0     # not configured: nothing to mirror (every rank has the same configuration)
        self.ch.send_desc(OP_DESCENT)
        return self.inner.kv_descent_step()

    def ping(self) -> bool:
        """Round trip over the control channel: every rank is in its loop and answers."""
        self.ch.send_desc(OP_PING)
        return self.ch.and_reduce(True)

    def shutdown(self) -> None:
        try:
            self.ch.send_desc(OP_STOP)
        except ResourceError:
            pass   # the followers are gone already


def _try_open(inner, prompt, sampling, session):
    try:
        return inner.open(prompt, sampling, session=session), None
    except RequestError as e:
        return None, f"request:{e}"
    except Exception as e:  # noqa: BLE001 - MemoryError, device errors: resource domain
        return None, f"resource:{type(e).__name__}: {e}"


def follower_loop(inner, channel: RankChannel, on_step: Optional[Callable[[int], None]] = None) -> str:
    """Executes the leader's steps on this rank's Program until it is told to stop.  Returns "stopped", or raises
    ResourceError when the channel fails (the leader or another rank is gone).  `on_step(op)` runs before each
    step is executed (tests use it to leave or to fail at a chosen point)."""
    while True:
        op, a = channel.recv_desc()
        if on_step is not None:
            on_step(op)
        if op == OP_STOP:
            return "stopped"
        if op == OP_PING:
            channel.and_reduce(True)
        elif op == OP_CAN_ADMIT:
            channel.and_reduce(inner.can_admit(int(a[0]), int(a[1])))
        elif op == OP_OPEN:
            prompt, sp, session, lane_id = channel.bcast_object()
            inner._next_id = int(lane_id)
            lane, err = _try_open(inner, prompt, _sampling_from_wire(sp), session)
            errs = channel.gather_errors(err)
            if any(e is not None for e in errs) and lane is not None:
                inner.close(lane)
        elif op == OP_CLOSE:
            lane = inner.lanes.get(int(a[0]))
            if lane is not None:
                inner.close(lane)
        elif op == OP_PREFILL:
            try:
                inner.prefill_step(inner.lanes[int(a[0])], int(a[1]))
            except RequestError:
                pass   # the leader hit the same refusal and closes the lane with its next step
        elif op == OP_DECODE:
            inner.decode_round([inner.lanes[int(i)] for i in a])
        elif op == OP_DESCENT:
            inner.kv_descent_step()
        elif op == OP_FORCE:
            lane = inner.lanes.get(int(a[0]))
            if lane is not None:
                inner.force_next_token(lane, int(a[1]))
        elif op == OP_CHECKPOINT:
            session = channel.bcast_object()
            inner.checkpoint(inner.lanes[int(a[0])], session, _KINDS[int(a[1])])
        else:
            raise ResourceError(f"unknown step descriptor {op}")
