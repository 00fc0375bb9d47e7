"""Multi-rank engine with PARTITIONED lanes: every request lives on one rank, one leader schedules all of them.

`parallel.replicated` runs the same lanes on every rank (tensor parallelism: a request's tokens are needed
everywhere).  Under expert parallelism the dense part of the model is replicated and only the routed experts are
sharded, so a request's attention / GDN work belongs on ONE rank (data parallel) while every MoE layer exchanges
tokens between all ranks.  That is this module:

* The leader (rank 0) owns the `Engine` and the front end.  Its Program is a `PartitionedLeader`: lanes are proxies that
  remember their owner rank; admission picks the rank with the most free lanes and asks THAT rank whether the request
  fits; every verb is broadcast as one small message and answered with one all-gather, so a rank that stops answering
  turns the next verb into a time-out (`ResourceError`, engine-wide failure, `recover()`), never into a hang.
* Every rank (the leader included) executes the verbs that concern its own lanes on its own Program.
* **Lock step** (needed when the ranks meet inside every forward pass, i.e. expert parallelism): each verb that runs
  a forward pass on some rank runs exactly one forward pass on EVERY rank.  A rank with nothing to do for that verb
  decodes one token of a scratch lane and rolls the lane's length back, so that its cache does not grow; the bound on
  the step's tokens over all ranks (`set_global_tokens`, the MoE kernels size their exchange by it) travels with the
  verb.  Without lock step (plain data parallel replicas) idle ranks just skip the verb.

The reference has no multi-GPU product path (its multi-device code is a set of host-proved contracts,
docs/maintainer/multi-device-and-shard-plan.md:111-160: replicated decisions, one decision maker); this is the
data-parallel + expert-parallel plan those contracts leave room for.  Tested on CPU with gloo ranks
(tests/test_partitioned_cpu.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch.distributed as dist

from ..runtime.engine import RequestError, ResourceError
from .replicated import RankChannel, _sampling_from_wire, _sampling_to_wire


@dataclass
class ProxyLane:
    """The leader's view of a lane that lives on `owner`."""
    lane_id: int
    owner: int
    tokens: List[int] = field(default_factory=list)
    n_cached: int = 0
    last_token: int = -1
    reused: int = 0
    reuse_kind: str = ""
    sampling: object = None
    row: int = -1
    slot: int = -1
    reserved_tokens: int = 0


class _Worker:
    """One rank's side: its Program, its lanes by global id, its scratch lane for lock-step filler passes."""

    def __init__(self, inner, rank: int, world: int, lockstep: bool):
        self.inner, self.rank, self.world, self.lockstep = inner, rank, world, lockstep
        self.lanes: Dict[int, object] = {}
        self.scratch = None
        self.filler_steps = 0
        self.forward_steps = 0

    def start(self) -> None:
        """Lock step: every rank prefills its one-token scratch lane at the same moment (one forward pass each)."""
        if not self.lockstep:
            return
        self._bound(self.world)
        self.scratch = self.inner.open([0], None, session=None)
        self.inner.prefill_step(self.scratch, 1)
        self.forward_steps += 1

    def _bound(self, n_tokens: int) -> None:
        f = getattr(self.inner, "set_global_tokens", None)
        if f is not None:
            f(int(n_tokens))

    def _filler(self) -> None:
        """One forward pass that changes nothing a request can see: decode the scratch lane, roll its length back."""
        s = self.scratch
        n, toks, last = s.n_cached, len(s.tokens), s.last_token
        self.inner.decode_round([s])
        s.n_cached, s.last_token = n, last
        del s.tokens[toks:]
        self.filler_steps += 1
        self.forward_steps += 1

    def execute(self, msg: dict):
        """This rank's part of one verb.  Returns (reply, error text or None)."""
        op = msg["op"]
        mine = msg.get("owner") == self.rank
        try:
            if op == "can_admit":
                return (self.inner.can_admit(msg["n_prompt"], msg["max_new"]) if mine else None), None
            if op == "open":
                if not mine:
                    return None, None
                lane = self.inner.open(msg["prompt"], _sampling_from_wire(msg["sampling"]), session=msg["session"])
                reserve = getattr(self.inner, "reserve", None)
                if reserve is not None and msg.get("reserve"):
                    reserve(lane, msg["reserve"])
                self.lanes[msg["lane"]] = lane
                return {"n_cached": lane.n_cached, "reused": lane.reused, "reuse_kind": lane.reuse_kind}, None
            if op == "reserve":
                f = getattr(self.inner, "reserve", None)
                if mine and f is not None:
                    f(self.lanes[msg["lane"]], msg["tokens"])
                return None, None
            if op == "force":
                if mine:
                    self.inner.force_next_token(self.lanes[msg["lane"]], msg["token"])
                return None, None
            if op == "close":
                lane = self.lanes.pop(msg["lane"], None) if mine else None
                if lane is not None:
                    self.inner.close(lane)
                return None, None
            if op == "checkpoint":
                if not mine:
                    return None, None
                return bool(self.inner.checkpoint(self.lanes[msg["lane"]], msg["session"], msg["kind"])), None
            if op == "prefill":
                self._bound(msg["bound"])
                if mine:
                    lane = self.lanes[msg["lane"]]
                    first = self.inner.prefill_step(lane, msg["budget"])
                    self.forward_steps += 1
                    return {"first": first, "n_cached": lane.n_cached, "last_token": lane.last_token}, None
                if self.lockstep:
                    self._filler()
                return None, None
            if op == "decode":
                self._bound(msg["bound"])
                ids = msg["lanes"].get(self.rank, [])
                if ids:
                    lanes = [self.lanes[i] for i in ids]
                    toks = self.inner.decode_round(lanes)
                    self.forward_steps += 1
                    return {i: (t, l.n_cached, l.last_token) for i, t, l in zip(ids, toks, lanes)}, None
                if self.lockstep:
                    self._filler()
                return {}, None
            if op == "descent":
                f = getattr(self.inner, "kv_descent_step", None)
                return (f() if f is not None else 0), None
            if op == "ping":
                return True, None
            raise ResourceError(f"unknown verb {op!r}")
        except RequestError as e:
            return None, f"request:{e}"
        except ResourceError:
            raise
        except Exception as e:  # noqa: BLE001 - MemoryError, device errors: resource domain
            return None, f"resource:{type(e).__name__}: {e}"


def _exchange(ch: RankChannel, worker: _Worker, msg: Optional[dict]):
    """One verb: the leader's message reaches every rank, every rank runs its part, all replies reach every rank."""
    msg = ch.bcast_object(msg)
    if msg["op"] == "stop":
        return msg, [], []
    reply, err = worker.execute(msg)
    box: List[object] = [None] * ch.world
    ch._collective(lambda: dist.all_gather_object(box, (reply, err), group=ch.group))
    return msg, [b[0] for b in box], [b[1] for b in box]


def _raise_first(errs: Sequence[Optional[str]], what: str) -> None:
    bad = [(r, e) for r, e in enumerate(errs) if e is not None]
    if not bad:
        return
    r, e = bad[0]
    kind, _, text = e.partition(":")
    exc = RequestError if all(b[1].startswith("request:") for b in bad) else ResourceError
    raise exc(f"rank {r} {what}: {text}")


class PartitionedLeader:
    """The Program the leader's Engine talks to."""

    supports_media = False

    def __init__(self, inner, channel: RankChannel, lanes_per_rank: int, lockstep: bool = True):
        self.ch = channel
        self.worker = _Worker(inner, channel.rank, channel.world, lockstep)
        self.lockstep = lockstep
        self.max_context = inner.max_context
        self.lanes_per_rank = lanes_per_rank - (1 if lockstep else 0)    # one lane per rank is the scratch lane
        if self.lanes_per_rank < 1:
            raise ValueError("lock step needs at least two lanes per rank (one is the scratch lane)")
        self.lanes: Dict[int, ProxyLane] = {}
        self._next_id = 0
        self._owner_for_next: Optional[int] = None
        self.partition_stats = {"verbs": 0, "per_rank_opened": [0] * channel.world}
        self.worker.start()

    # ---- read-only surface ----
    @property
    def device_wait_s(self) -> float:
        return float(getattr(self.worker.inner, "device_wait_s", 0.0))

    @property
    def anchor_interval(self) -> int:
        return int(getattr(self.worker.inner, "anchor_interval", 0))

    def _load(self) -> List[int]:
        n = [0] * self.ch.world
        for l in self.lanes.values():
            n[l.owner] += 1
        return n

    def free_lanes(self) -> int:
        return sum(self.lanes_per_rank - n for n in self._load())

    def census(self) -> dict:
        c = self.worker.inner.census() if hasattr(self.worker.inner, "census") else {}
        c["ranks"] = self.ch.world
        c["partitioned"] = dict(self.partition_stats, lanes_per_rank=self.lanes_per_rank, load=self._load(),
                                lockstep=self.lockstep, filler_steps=self.worker.filler_steps)
        return c

    def _verb(self, msg: dict):
        self.partition_stats["verbs"] += 1
        _, replies, errs = _exchange(self.ch, self.worker, msg)
        return replies, errs

    # ---- Program API ----
    def can_admit(self, n_prompt: int, max_new: int) -> bool:
        if n_prompt + max_new > self.max_context:
            return False
        load = self._load()
        order = sorted(range(self.ch.world), key=lambda r: (load[r], r))
        for owner in order:                       # least loaded first; ask the rank itself whether its pages allow it
            if load[owner] >= self.lanes_per_rank:
                break
            replies, errs = self._verb({"op": "can_admit", "owner": owner, "n_prompt": n_prompt, "max_new": max_new})
            _raise_first(errs, "could not answer the admission check")
            if replies[owner]:
                self._owner_for_next = owner
                return True
        return False

    def open(self, prompt, sampling=None, session=None, media=None):
        if media is not None:
            raise RequestError("media prompts are not supported by the partitioned multi-rank engine")
        owner = self._owner_for_next
        if owner is None:
            load = self._load()
            owner = min(range(self.ch.world), key=lambda r: (load[r], r))
        self._owner_for_next = None
        gid = self._next_id
        self._next_id += 1
        replies, errs = self._verb({"op": "open", "owner": owner, "lane": gid, "prompt": list(prompt),
                                    "sampling": _sampling_to_wire(sampling), "session": session, "reserve": 0})
        _raise_first(errs, "could not open the lane")
        r = replies[owner]
        lane = ProxyLane(gid, owner, list(prompt), r["n_cached"], -1, r["reused"], r["reuse_kind"], sampling)
        self.lanes[gid] = lane
        self.partition_stats["per_rank_opened"][owner] += 1
        return lane

    def reserve(self, lane: ProxyLane, n_tokens: int) -> None:
        lane.reserved_tokens = int(n_tokens)
        _, errs = self._verb({"op": "reserve", "owner": lane.owner, "lane": lane.lane_id, "tokens": int(n_tokens)})
        _raise_first(errs, "could not reserve the request's pages")

    def force_next_token(self, lane: ProxyLane, token: int) -> None:
        lane.last_token = int(token)
        _, errs = self._verb({"op": "force", "owner": lane.owner, "lane": lane.lane_id, "token": int(token)})
        _raise_first(errs, "could not replace the next token")

    def close(self, lane: ProxyLane) -> None:
        if self.lanes.pop(lane.lane_id, None) is None:
            return
        self._verb({"op": "close", "owner": lane.owner, "lane": lane.lane_id})

    def checkpoint(self, lane: ProxyLane, session, kind: str) -> bool:
        replies, errs = self._verb({"op": "checkpoint", "owner": lane.owner, "lane": lane.lane_id, "session": session,
                                    "kind": kind})
        _raise_first(errs, "could not keep the frontier")
        return bool(replies[lane.owner])

    def prefill_step(self, lane: ProxyLane, budget: int):
        left = len(lane.tokens) - lane.n_cached
        bound = min(int(budget), left) + (self.ch.world - 1)      # the owner's chunk + one filler token per other rank
        replies, errs = self._verb({"op": "prefill", "owner": lane.owner, "lane": lane.lane_id, "budget": int(budget),
                                    "bound": bound})
        _raise_first(errs, "failed in a prefill step")
        r = replies[lane.owner]
        lane.n_cached = r["n_cached"]
        if r["first"] is not None:
            lane.last_token = r["last_token"]
        return r["first"]

    def decode_round(self, lanes: Sequence[ProxyLane]):
        by_rank: Dict[int, List[int]] = {}
        for l in lanes:
            by_rank.setdefault(l.owner, []).append(l.lane_id)
        # a constant bound under lock step: a captured decode graph bakes the sizes derived from it, and the other
        # ranks' lane counts change from round to round
        bound = (self.ch.world * (self.lanes_per_rank + 1) if self.lockstep
                 else sum(max(1, len(by_rank.get(r, []))) for r in range(self.ch.world)))
        replies, errs = self._verb({"op": "decode", "lanes": by_rank, "bound": bound})
        _raise_first(errs, "failed in a decode round")
        out = []
        for l in lanes:
            tok, n_cached, last = replies[l.owner][l.lane_id]
            new = list(tok) if isinstance(tok, (list, tuple)) else [tok]
            l.tokens.append(l.last_token)
            l.tokens.extend(new[:-1])
            l.n_cached, l.last_token = n_cached, last
            out.append(tok)
        return out

    def kv_descent_step(self) -> int:
        if getattr(self.worker.inner, "descent", None) is None:
            return 0
        replies, errs = self._verb({"op": "descent"})
        _raise_first(errs, "failed in the KV descent step")
        return int(sum(r or 0 for r in replies))

    def ping(self) -> bool:
        replies, errs = self._verb({"op": "ping"})
        return all(replies) and not any(errs)

    def shutdown(self) -> None:
        try:
            self.ch.bcast_object({"op": "stop"})
        except ResourceError:
            pass


def partitioned_follower_loop(inner, channel: RankChannel, lockstep: bool = True,
                              on_verb: Optional[Callable[[dict], None]] = None) -> _Worker:
    """A follower's life: run this rank's part of every verb until the leader says stop.  Returns the worker (its
    counters) when stopped; raises ResourceError when the channel fails.  `on_verb(msg)` runs after a verb was received
    and before it is executed (tests use it to leave or to fail at a chosen point)."""
    worker = _Worker(inner, channel.rank, channel.world, lockstep)
    worker.start()
    while True:
        msg = channel.bcast_object(None)
        if msg["op"] == "stop":
            return worker
        if on_verb is not None:
            on_verb(msg)
        reply, err = worker.execute(msg)
        box: List[object] = [None] * channel.world
        channel._collective(lambda: dist.all_gather_object(box, (reply, err), group=channel.group))
