"""Program: the physical layer under the engine (lanes, KV rows, GDN slots, graphs, sampling).

A *lane* is one live sequence: a KV block-table row, a GDN state slot, its token history and its
sampling state.  The engine drives three verbs -- `prefill_step` (advance one lane by a chunk),
`decode_round` (one token for every listed lane, exact batch size, CUDA graph per (B, context bucket,
sampler kind)) and `close` -- plus `fork` / `snapshot` for prefix reuse.  This is the counterpart of the
reference's `Program<Variant>` surface (src/targets/qwen3_6/export/ninfer/targets/qwen3_6/runtime.h:739-905:
plan_request / advance_prefill / decode / commit / finish) with one deliberate difference: batch sizes
are not capped at 16 lanes, because the B200 configurations ask for 32..128 concurrent sequences.

`ReferenceProgram` implements the same verbs on the pure-PyTorch CPU oracle, so the engine, the
scheduler and the gateways can be tested end to end without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..models.config import ModelConfig
from ..ops import reference as R


@dataclass
class SamplingParams:
    temperature: float = 0.0          # <= 0: greedy
    top_k: int = 20
    top_p: float = 1.0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


@dataclass
class Lane:
    lane_id: int
    row: int                 # KV block-table row
    slot: int                # GDN state slot
    tokens: List[int] = field(default_factory=list)   # every token whose KV/state is (or will be) materialised
    n_cached: int = 0        # tokens already run through the model
    sampling: SamplingParams = field(default_factory=SamplingParams)
    last_token: int = -1     # sampled but not yet fed
    reused: int = 0          # prompt tokens restored from a session checkpoint instead of being prefilled
    reuse_kind: str = ""     # kind of the frontier those tokens came from ("" = none: the request started at the root)
    media: object = None     # frontend.media.PreparedPrompt of a multimodal request
    visual: object = None    # [V, hidden] vision-tower output of `media` (filled at the first prefill step)
    rope_delta: int = 0      # rope position - cache position once the prompt is in (multimodal prompts)
    reserved_tokens: int = 0  # cache positions this request may still grow into (prompt + generation budget)
    session: Optional[str] = None  # continuation key of the request on this lane (its session is "live" meanwhile)


@dataclass
class Checkpoint:
    """A reusable frontier of a session: exact token history + KV coverage + recurrent state image.
    Kinds follow the reference's catalogue (docs/maintainer/resource-scheduling-and-context-cache.md:266-284):
    'turn' = the prompt boundary of a request (TurnClosure), 'endpoint' = where its generation stopped
    (SessionEndpoint), 'replay' = the history before the generation opener (ResponseReplay), 'anchor' = an earlier
    recovery point inside a long prompt (LongAnchor), 'shared' = an immutable
    prefix any session may start from (SharedStablePrefix).  A frontier is reusable only for a prompt that starts with exactly these tokens."""
    session: str
    kind: str
    tokens: List[int]
    handle: object
    last_used: float = 0.0
    tier: str = "gpu"     # "gpu" | "host" | "disk": where the KV pages and the state image currently live
    nbytes: int = 0       # size of the cold copy (host / disk tiers)
    hits: int = 0         # times a request started from this frontier (the planner's demand signal)


SHARED_SESSION = "__shared__"

# Retention classes of reusable frontiers and the weight each carries when a victim is chosen (a frontier of weight w
# is given up before one of weight > w; shared prefixes live in their own bounded catalogue and are only taken when no
# private frontier is left).  Reference: RetentionClass in src/runtime/contract/types.h:383-388 and
# ResourceManager::private_retention_weight (src/runtime/engine/resource_manager.h:1298-1310).
RETENTION_WEIGHT = {"disposable": 1, "recent_private": 4, "live_session": 16, "shared_stable": 0}


class ProgramBase:
    """Lane bookkeeping shared by the GPU and the CPU-reference programs."""

    def __init__(self, cfg: ModelConfig, max_lanes: int, max_context: int):
        self.cfg = cfg
        self.max_lanes = max_lanes
        self.max_context = max_context
        self.lanes: Dict[int, Lane] = {}
        self._free_rows = list(range(max_lanes - 1, -1, -1))
        self._next_id = 0
        self.checkpoints: List[Checkpoint] = []
        self.max_checkpoints = 2 * max_lanes
        self._clock = 0
        # cold tiers for session checkpoints: frontiers pushed out of the device pool are parked in pinned host memory
        # and, beyond that budget, in files (host_budget_bytes = 0 keeps the old "evict = drop" behaviour)
        self.host_budget_bytes = 0
        self.disk_budget_bytes = 0
        self.cold_dir: Optional[str] = None
        self.cold_entropy = False   # entropy-code frontiers written to the disk tier (kv/cold_codec.py)
        self.cold_stats = {"demoted_host": 0, "demoted_disk": 0, "promoted": 0, "dropped": 0}
        # persistent map frontier -> disk file (runtime/cold_journal.py): off until enable_cold_journal()
        self.cold_journal = None
        self.recall_cost = None     # RecallCost: read a disk frontier back only when that beats prefilling it again
        self._cold_nonce = ""
        # shared-prefix catalogue: frontiers of prompt prefixes that any request may start from (system prompts)
        self.max_shared_prefixes = 8
        # long anchors: while a long prompt is prefilled, a frontier is kept every `anchor_interval` tokens (0 = off) so
        # that a later request of the session whose history DIVERGES part-way (an edited turn) restarts from the last
        # anchor before the edit instead of from zero; at most `max_anchors` per session, thinned to stay spread out
        self.anchor_interval = 0
        self.max_anchors = 3
        self.shared_stats = {"published": 0, "hits": 0}
        self.device_wait_s = 0.0   # wall time this program's steps spent blocked on the device (the engine reads deltas)

    # ---- capacity ----
    def free_lanes(self) -> int:
        return len(self._free_rows)

    def can_admit(self, n_prompt: int, max_new: int) -> bool:
        if not self._free_rows or n_prompt + max_new > self.max_context:
            return False
        while not self._kv_room(n_prompt + max_new):
            if not self._evict_checkpoint():   # cached frontiers give way to live requests, oldest first
                return False
        return True

    # ---- page reservations and the admission proof ----
    # A program with a page pool overrides the three hooks; the base (no pool) never runs short.
    def _pages_for(self, n_tokens: int) -> int:
        return 0

    def _pages_free(self) -> int:
        return 1 << 60

    def _pages_held(self, lane: Lane) -> int:
        return 0

    def reserve(self, lane: Lane, n_tokens: int) -> None:
        """The request on `lane` may grow to `n_tokens` cache positions: the pages it has not taken yet are no longer
        free for admission (pages are handed out step by step, so without this two requests could each be admitted
        against the same free pages and run out half-way)."""
        lane.reserved_tokens = max(lane.reserved_tokens, int(n_tokens))

    def outstanding_reservation(self) -> int:
        """Pages that admitted requests are still entitled to take."""
        return sum(max(0, self._pages_for(l.reserved_tokens) - self._pages_held(l)) for l in self.lanes.values())

    def pages_available(self) -> int:
        return self._pages_free() - self.outstanding_reservation()

    def admission_proof(self, head_tokens: int, candidate_tokens: int, donors: Sequence[Lane]) -> bool:
        """May a request of `candidate_tokens` positions be admitted ahead of a blocked head of `head_tokens`?  Yes if
        it fits now and the head still fits once every donor lane has left while the candidate is still resident
        (the donors give back their whole reservation and their lanes; cached frontiers are not counted: they can
        only add room)."""
        need_c, need_h = self._pages_for(candidate_tokens), self._pages_for(head_tokens)
        free = self.pages_available()
        if not self._free_rows or free < need_c:
            return False
        live = [l for l in donors if l.lane_id in self.lanes]
        released = sum(max(self._pages_for(l.reserved_tokens), self._pages_held(l)) for l in live)
        lanes_then = len(self._free_rows) - 1 + len(live)
        pages_then = free - need_c + released
        return lanes_then >= 1 and pages_then >= need_h

    # ---- census ----
    def census(self) -> dict:
        """Where the reusable state lives right now: frontiers per tier and kind, bytes of the cold copies, page pool
        occupancy and bytes per KV plane format when the program has a paged cache (residency / plane census of the
        reference: src/product/kv_residency_census.h, kv_plane_census.h)."""
        tiers = {"gpu": 0, "host": 0, "disk": 0}
        kinds: dict = {}
        cold_bytes = {"host": 0, "disk": 0}
        for c in self.checkpoints:
            tiers[c.tier] = tiers.get(c.tier, 0) + 1
            kinds[c.kind] = kinds.get(c.kind, 0) + 1
            if c.tier in cold_bytes:
                cold_bytes[c.tier] += c.nbytes
        out = {"lanes": {"active": len(self.lanes), "max": self.max_lanes}, "frontiers": tiers, "kinds": kinds,
               "cold_bytes": cold_bytes, "budgets": {"host": self.host_budget_bytes, "disk": self.disk_budget_bytes},
               "cold_stats": dict(self.cold_stats), "shared_stats": dict(self.shared_stats)}
        retention = {k: 0 for k in RETENTION_WEIGHT}
        for c in self.checkpoints:
            retention[self.retention_class(c)] += 1
        out["retention"] = retention                                  # counts only: no session names leave the engine
        out["sessions"] = len({c.session for c in self.checkpoints if c.session != SHARED_SESSION})
        kv = getattr(self, "kv", None)
        pool = getattr(kv, "pool", None)
        if pool is not None:
            free = int(getattr(pool, "free_pages", 0))
            out["pages"] = {"total": int(kv.n_pages), "free": free, "used": int(kv.n_pages) - free,
                            "page_tokens": int(kv.page_size)}
            planes: dict = {}
            for l in kv.layers:
                planes[l.fmt] = planes.get(l.fmt, 0) + int(l.bytes())
            out["plane_bytes_by_format"] = planes
        return out

    # ---- session checkpoints (prefix reuse) ----
    def _evict_checkpoint(self) -> bool:
        """Frees the device resources of the least recently used device-resident frontier: it is demoted to the host
        tier when the budget allows (pushing older host copies on to disk), otherwise dropped."""
        hot = [c for c in self.checkpoints if c.tier == "gpu"]
        if not hot:
            return False
        victim = self._choose_victim(hot)
        cold = self._demote(victim.handle) if self.host_budget_bytes > 0 else None
        self._drop(victim.handle)
        if cold is None:
            self.checkpoints.remove(victim)
            self.cold_stats["dropped"] += 1
            return True
        victim.handle, victim.tier, victim.nbytes = cold, "host", self._cold_bytes(cold)
        self.cold_stats["demoted_host"] += 1
        self._trim_cold()
        return True

    def retention_class(self, c: Checkpoint) -> str:
        """shared_stable: an entry of the shared-prefix catalogue.  live_session: a request of the frontier's session
        is on a lane right now (its next turn is the most likely one to arrive).  disposable: a longer frontier of
        the same session extends this one, so only an edited history would still want it.  recent_private: the rest."""
        if c.kind == "shared" or c.session == SHARED_SESSION:
            return "shared_stable"
        n = len(c.tokens)
        # the latest replay frontier of a session is where "regenerate this response" restarts: the turn frontier
        # that extends it by the generation opener does not make it disposable
        regenerate_point = c.kind == "replay" and not any(
            o.kind == "replay" and o.session == c.session and len(o.tokens) > n for o in self.checkpoints)
        if not regenerate_point:
            for o in self.checkpoints:
                if o is not c and o.session == c.session and len(o.tokens) > n and o.tokens[:n] == c.tokens:
                    return "disposable"
        if any(l.session == c.session for l in self.lanes.values()):
            return "live_session"
        return "recent_private"

    def session_index(self) -> Dict[str, dict]:
        """Session -> what is kept for it: number of frontiers, the longest one, where it lives, its retention class."""
        out: Dict[str, dict] = {}
        for c in self.checkpoints:
            if c.session == SHARED_SESSION:
                continue
            e = out.setdefault(c.session, {"frontiers": 0, "longest_tokens": 0, "tier": "", "retention": "", "hits": 0})
            e["frontiers"] += 1
            e["hits"] += c.hits
            if len(c.tokens) >= e["longest_tokens"]:
                e["longest_tokens"], e["tier"], e["retention"] = len(c.tokens), c.tier, self.retention_class(c)
        return out

    def _choose_victim(self, hot: List[Checkpoint]) -> Checkpoint:
        private = [c for c in hot if self.retention_class(c) != "shared_stable"]
        if private:
            low = min(RETENTION_WEIGHT[self.retention_class(c)] for c in private)
            hot = [c for c in private if RETENTION_WEIGHT[self.retention_class(c)] == low]
        return self._cheapest_loss(hot)

    def _cheapest_loss(self, hot: List[Checkpoint]) -> Checkpoint:
        """Least recently used without a planner; with one (`self.planner`, runtime/planner.py) the frontier whose loss
        costs least per token of context it holds: demand (hits, recency, shared credit) times the cost of getting
        it back from the tier it would fall to."""
        planner = getattr(self, "planner", None)
        if planner is None:
            return min(hot, key=lambda c: c.last_used)
        from .planner import DROP, TO_HOST, Owner
        action = TO_HOST if self.host_budget_bytes > 0 else DROP

        def loss(c: Checkpoint) -> float:
            n = max(1, len(c.tokens))
            o = Owner(key=id(c), pages=n, tokens=n, nbytes=n * getattr(self, "bytes_per_token_estimate", 65536),
                      hits=c.hits, last_hit_epoch=int(c.last_used), shared=c.session == SHARED_SESSION)
            return planner.action_cost(o, action, self._clock) / n
        return min(hot, key=lambda c: (loss(c), c.last_used))

    def _cold_bytes(self, cold) -> int:
        return sum(t.numel() * t.element_size() for group in cold["tensors"] for t in group)

    def _trim_cold(self) -> None:
        """Keeps the host tier inside its budget: oldest host copies go to disk (or are dropped without a disk tier)."""
        import os
        while sum(c.nbytes for c in self.checkpoints if c.tier == "host") > self.host_budget_bytes:
            victim = min((c for c in self.checkpoints if c.tier == "host"), key=lambda c: c.last_used)
            on_disk = sum(c.nbytes for c in self.checkpoints if c.tier == "disk")
            if self.cold_dir and on_disk + victim.nbytes <= self.disk_budget_bytes:
                path = os.path.join(self.cold_dir, f"ckpt_{id(victim):x}_{self._clock}{self._cold_nonce}.pt")
                try:
                    os.makedirs(self.cold_dir, exist_ok=True)
                    if self.cold_entropy and set(victim.handle) == {"n_pages", "tensors"}:
                        # lossless entropy stage (rANS per tensor, raw when it does not pay): fewer bytes on disk
                        from ..kv.cold_codec import save_cold
                        st = save_cold(victim.handle, path)
                        self.cold_stats["disk_raw_bytes"] = self.cold_stats.get("disk_raw_bytes", 0) + st["raw"]
                        self.cold_stats["disk_stored_bytes"] = self.cold_stats.get("disk_stored_bytes", 0) + st["stored"]
                    else:
                        torch.save(victim.handle, path)
                except OSError:
                    # a spill that cannot be written (full or read-only disk) costs this frontier, not the engine:
                    # it is counted and the copy is dropped (the reference counts cold-spill write failures the same way)
                    self.cold_stats["spill_write_failed"] = self.cold_stats.get("spill_write_failed", 0) + 1
                    try:
                        os.remove(path)
                    except OSError:
                        pass
                    self.checkpoints.remove(victim)
                    self.cold_stats["dropped"] += 1
                    continue
                victim.handle, victim.tier = {"path": path}, "disk"
                self.cold_stats["demoted_disk"] += 1
                if self.cold_journal is not None:
                    from .cold_journal import SpillRecord
                    self.cold_journal.spill(SpillRecord(os.path.basename(path), victim.nbytes, os.path.getsize(path),
                                                        victim.session, victim.kind, list(victim.tokens)))
            else:
                self.checkpoints.remove(victim)
                self.cold_stats["dropped"] += 1
        while self.cold_dir and sum(c.nbytes for c in self.checkpoints if c.tier == "disk") > self.disk_budget_bytes:
            victim = min((c for c in self.checkpoints if c.tier == "disk"), key=lambda c: c.last_used)
            self._forget_cold(victim)

    def _forget_cold(self, c: Checkpoint) -> None:
        import os
        if c.tier == "disk":
            self._release_cold_file(c.handle["path"], "dropped")
        self.checkpoints.remove(c)
        self.cold_stats["dropped"] += 1

    def _release_cold_file(self, path: str, reason: str) -> None:
        import os
        try:
            os.remove(path)
        except OSError:
            pass
        if self.cold_journal is not None:
            self.cold_journal.release(os.path.basename(path), reason)

    def _warm_up(self, c: Checkpoint) -> bool:
        """Brings a cold frontier back into the device pool (disk -> host -> device).  False if there is no room."""
        if c.tier == "gpu":
            return True
        if c.tier == "disk" and self.recall_cost is not None and not self.recall_cost.worthwhile(c.nbytes, len(c.tokens)):
            return False     # prefilling these tokens again is faster than reading their cold copy
        try:
            cold = self._read_cold_file(c.handle["path"]) if c.tier == "disk" else c.handle
        except Exception:
            # a cold file that cannot be read back (damaged, truncated, gone) costs this frontier, not the request
            self.cold_stats["read_failed"] = self.cold_stats.get("read_failed", 0) + 1
            self._forget_cold(c)
            return False
        handle = self._promote(cold)
        while handle is None:
            others = [o for o in self.checkpoints if o.tier == "gpu" and o is not c]
            if not others or not self._evict_checkpoint():
                return False
            handle = self._promote(cold)
        if c.tier == "disk":
            self._release_cold_file(c.handle["path"], "promoted")
        c.handle, c.tier, c.nbytes = handle, "gpu", 0
        self.cold_stats["promoted"] += 1
        return True

    def cold_fingerprint(self, weights_id: str = "") -> str:
        """What a cold copy is only valid for: this program class, model geometry, KV storage and set of weights."""
        cfg = self.cfg
        kv = getattr(self, "kv_layer_formats", None) or getattr(self, "kv_dtype", "") or "reference"
        return "|".join(str(x) for x in (type(self).__name__, cfg.name, cfg.n_layers, cfg.hidden, cfg.n_kv_heads, cfg.head_dim,
                                         kv, weights_id))

    def enable_cold_journal(self, weights_id: str = "", flush: str = "none", remove_orphans: bool = True) -> dict:
        """Keeps the disk tier's frontier -> file map in a journal inside the cold directory and adopts the frontiers
        a previous process left there: each becomes a disk-tier frontier of its session again, reusable for a prompt
        that starts with exactly its tokens.  Returns what was found."""
        import os
        from .cold_journal import ColdJournal
        if not self.cold_dir or self.disk_budget_bytes <= 0:
            raise ValueError("the cold journal needs a disk tier (a cold directory and a byte budget)")
        self._cold_nonce = "_" + os.urandom(4).hex()      # file names of this process never collide with adopted ones
        j = ColdJournal(self.cold_dir, self.cold_fingerprint(weights_id), flush)
        self.cold_journal = j
        good, holes = j.adoptable()
        adopted = skipped = 0
        on_disk = sum(c.nbytes for c in self.checkpoints if c.tier == "disk")
        for r in sorted(good, key=lambda r: -len(r.tokens)):
            if on_disk + r.nbytes > self.disk_budget_bytes:
                self._release_cold_file(os.path.join(self.cold_dir, r.file), "over budget at adoption")
                skipped += 1
                continue
            self.checkpoints.append(Checkpoint(r.session, r.kind, list(r.tokens), {"path": os.path.join(self.cold_dir, r.file)},
                                               0.0, "disk", r.nbytes))
            on_disk += r.nbytes
            adopted += 1
        orphans = j.orphans() if remove_orphans else []
        for name in orphans:
            try:
                os.remove(os.path.join(self.cold_dir, name))
            except OSError:
                pass
        self.cold_stats["adopted"] = self.cold_stats.get("adopted", 0) + adopted
        return {"adopted": adopted, "over_budget": skipped, "holes": holes, "orphans_removed": len(orphans),
                "refused": j.report.refused, "ignored_tail_bytes": j.report.ignored_tail_bytes, "records": j.report.records}

    @staticmethod
    def _read_cold_file(path: str):
        from ..kv.cold_codec import FILE_MAGIC, load_cold
        with open(path, "rb") as f:
            coded = f.read(len(FILE_MAGIC)) == FILE_MAGIC
        return load_cold(path) if coded else torch.load(path, weights_only=False)

    def _demote(self, handle):
        return None   # programs without a cold tier drop evicted frontiers

    def _promote(self, cold):
        return None

    def checkpoint(self, lane: Lane, session: str, kind: str) -> bool:
        """Remember the lane's materialised frontier (lane.tokens[:n_cached]) for `session`.

        kind 'shared' publishes the frontier in the shared-prefix catalogue (session SHARED_SESSION): any later request
        whose prompt starts with exactly these tokens may start from it, whatever its session.  The catalogue keeps
        `max_shared_prefixes` entries, least recently used first out; an identical prefix is only refreshed."""
        if lane.media is not None:
            return False   # see open(): multimodal histories are not reusable by token ids alone
        n = lane.n_cached
        if not session or n <= 0:
            return False
        if kind == "shared":
            session = SHARED_SESSION
            toks = list(lane.tokens[:n])
            shared = [c for c in self.checkpoints if c.kind == "shared"]
            for c in shared:
                if c.tokens == toks:
                    self._clock += 1
                    c.last_used = self._clock
                    return True
            while len(shared) >= self.max_shared_prefixes:
                victim = min(shared, key=lambda c: c.last_used)
                shared.remove(victim)
                if victim.tier == "gpu":
                    self.checkpoints.remove(victim)
                    self._drop(victim.handle)
                else:
                    self._forget_cold(victim)
        if kind == "anchor":
            anchors = sorted((c for c in self.checkpoints if c.session == session and c.kind == "anchor"),
                             key=lambda c: len(c.tokens))
            if any(len(c.tokens) == n for c in anchors):
                return True
            while len(anchors) >= self.max_anchors:
                # thin: drop the anchor whose neighbours are closest together (the coverage stays spread out)
                lens = [0] + [len(c.tokens) for c in anchors] + [n]
                i = min(range(len(anchors)), key=lambda j: lens[j + 2] - lens[j])
                victim = anchors.pop(i)
                if victim.tier == "gpu":
                    self.checkpoints.remove(victim)
                    self._drop(victim.handle)
                else:
                    self._forget_cold(victim)
                    self.cold_stats["dropped"] -= 1
        for c in [c for c in self.checkpoints if c.session == session and c.kind == kind and kind not in ("shared", "anchor")]:
            if c.tier == "gpu":              # one frontier per (session, kind)
                self.checkpoints.remove(c)
                self._drop(c.handle)
            else:
                self._forget_cold(c)
                self.cold_stats["dropped"] -= 1
        while len([c for c in self.checkpoints if c.tier == "gpu"]) >= self.max_checkpoints:
            self._evict_checkpoint()
        handle = None
        while handle is None:
            handle = self._snapshot(lane, n)
            if handle is None and not self._evict_checkpoint():
                return False
        self._clock += 1
        self.checkpoints.append(Checkpoint(session, kind, list(lane.tokens[:n]), handle, self._clock))
        if kind == "shared":
            self.shared_stats["published"] += 1
        return True

    def _match(self, session: Optional[str], prompt: Sequence[int]) -> Optional[Checkpoint]:
        best = None
        for c in self.checkpoints:
            n = len(c.tokens)
            mine = bool(session) and c.session == session
            if (mine or c.kind == "shared") and n < len(prompt) and (best is None or n > len(best.tokens)) \
                    and list(prompt[:n]) == c.tokens:
                best = c
        if best is not None and best.kind == "shared":
            self.shared_stats["hits"] += 1
        return best

    def _snapshot(self, lane: Lane, n_tokens: int):
        return None   # programs without checkpoint support simply never reuse

    def _restore(self, handle, lane: Lane, n_tokens: int) -> None:
        raise NotImplementedError

    def _drop(self, handle) -> None:
        pass

    def _kv_room(self, n_tokens: int) -> bool:
        return True

    supports_media = False
    supports_injection = False

    def open(self, prompt: Sequence[int], sampling: Optional[SamplingParams] = None,
             session: Optional[str] = None, media=None) -> Lane:
        if not self._free_rows:
            raise MemoryError("no free lane")
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        injected = media is not None and getattr(media, "rows", None) is not None and not getattr(media, "items", None)
        if injected:
            # rows of the embedding space at declared columns (runtime/inject.py): the multimodal mechanism without a tower
            if not self.supports_injection:
                raise ValueError("this program does not accept injected embedding rows")
            if list(media.ids) != list(prompt):
                raise ValueError("the injected prompt does not match the request's token ids")
            session = None   # frontiers are keyed by token ids only; injected rows are not part of that identity
        elif media is not None and getattr(media, "items", None):
            if not self.supports_media:
                raise ValueError("this program has no vision tower: media prompts are not supported")
            if list(media.ids) != list(prompt):
                raise ValueError("the prepared media prompt does not match the request's token ids")
            session = None   # frontiers are keyed by token ids only; visual content is not part of that identity
        else:
            media = None
        slot = self._alloc_slot()      # before the row is taken: a failure here must not leak the row
        row = self._free_rows.pop()
        lane = Lane(self._next_id, row, slot, list(prompt), 0, sampling or SamplingParams())
        if media is not None:
            lane.media, lane.rope_delta = media, int(media.rope_delta)
            if injected:
                lane.visual = media.rows
        lane.session = session
        self._next_id += 1
        self.lanes[lane.lane_id] = lane
        ck = self._match(session, prompt)
        if ck is not None and not self._warm_up(ck):
            ck = None   # no room to bring the cold frontier back: prefill from scratch
        if ck is not None:
            self._restore(ck.handle, lane, len(ck.tokens))
            lane.n_cached = lane.reused = len(ck.tokens)
            lane.reuse_kind = ck.kind
            self._clock += 1
            ck.last_used = self._clock
            ck.hits += 1
        return lane

    def force_next_token(self, lane: Lane, token: int) -> None:
        """The token that is fed next on `lane` instead of the one the last step sampled (that one has not been run
        through the model yet, so replacing it rewrites nothing)."""
        lane.last_token = int(token)

    def close(self, lane: Lane) -> None:
        if self.lanes.pop(lane.lane_id, None) is None:
            return
        self._release(lane)
        self._free_rows.append(lane.row)

    # ---- to be provided ----
    def _alloc_slot(self) -> int:
        raise NotImplementedError

    def _release(self, lane: Lane) -> None:
        raise NotImplementedError

    def prefill_step(self, lane: Lane, budget: int) -> Optional[int]:
        """Run up to `budget` not-yet-cached prompt tokens; returns the first sampled token when the prompt is done."""
        raise NotImplementedError

    def decode_round(self, lanes: Sequence[Lane]) -> List[int]:
        raise NotImplementedError


class ReferenceProgram(ProgramBase):
    """CPU program on the fp32 oracle model (tiny configurations only)."""
    supports_injection = True

    def __init__(self, cfg: ModelConfig, weights, max_lanes: int = 8, max_context: int = 4096, kv_format: str = "bf16"):
        super().__init__(cfg, max_lanes, max_context)
        from ..models.reference_model import ReferenceModel, ReferenceSequence

        self._Seq = ReferenceSequence
        self.model = ReferenceModel(cfg, weights)
        self.kv_fmt = R.KV_FORMAT_NAMES[kv_format]
        self._seqs: Dict[int, object] = {}
        self._slots = 0

    def _alloc_slot(self) -> int:
        self._slots += 1
        return self._slots

    def _release(self, lane: Lane) -> None:
        self._seqs.pop(lane.lane_id, None)

    def _snapshot(self, lane: Lane, n_tokens: int):
        import copy
        return copy.deepcopy(self._seqs[lane.lane_id])

    def _restore(self, handle, lane: Lane, n_tokens: int) -> None:
        import copy
        self._seqs[lane.lane_id] = copy.deepcopy(handle)

    def _demote(self, handle):
        seq = handle
        return {"n_pages": 0, "seq": seq, "tensors": [list(seq.k) + list(seq.v), list(seq.conv) + list(seq.ssm)]}

    def _promote(self, cold):
        return cold["seq"]

    def _sample(self, lane: Lane, logits: torch.Tensor) -> int:
        sp = lane.sampling
        lg = logits.float().clone()
        if sp.presence_penalty or sp.frequency_penalty:
            counts = torch.bincount(torch.tensor(lane.tokens), minlength=lg.numel()).float()
            lg -= (counts > 0).float() * sp.presence_penalty + counts * sp.frequency_penalty
        if sp.greedy:
            return int(R.argmax_lowest(lg[None])[0])
        k = sp.top_k if 0 < sp.top_k <= 32 else 32
        vals, idx = torch.sort(lg, descending=True, stable=True)
        vals, idx = vals[:k], idx[:k]
        p = torch.softmax((vals - vals[0]) / sp.temperature, 0)
        keep = (p >= sp.min_p * p[0]) if sp.min_p > 0 else torch.ones_like(p, dtype=torch.bool)
        p = p * keep
        p = p / p.sum()
        if sp.top_p < 1.0:
            c = torch.cumsum(p, 0)
            m = int((c < sp.top_p).sum().item()) + 1
            p[m:] = 0
            p = p / p.sum()
        g = torch.Generator().manual_seed((sp.seed * 1000003 + len(lane.tokens)) & 0x7FFFFFFF)
        return int(idx[int(torch.multinomial(p, 1, generator=g))])

    def attach_vision(self, vision_cfg, vision_weights) -> None:
        """Enables multimodal requests on the oracle program (fp32 vision tower on the CPU)."""
        if vision_cfg.out_hidden != self.cfg.hidden:
            raise ValueError("vision tower output width differs from the text hidden size")
        self._vision = (vision_cfg, vision_weights)
        self.supports_media = True

    def prefill_step(self, lane: Lane, budget: int) -> Optional[int]:
        seq = self._seqs.setdefault(lane.lane_id, self._Seq(self.cfg, self.kv_fmt))
        n = min(budget, len(lane.tokens) - lane.n_cached)
        ids = torch.tensor(lane.tokens[lane.n_cached:lane.n_cached + n])
        if lane.media is not None:
            import numpy as np
            from ..models.vision import build_control, vision_reference
            pm, c0 = lane.media, lane.n_cached
            if lane.visual is None:
                vcfg, vw = self._vision
                lane.visual = vision_reference(vcfg, vw, pm.patches(), build_control(pm.grids, vcfg.merge))
            lo, hi = np.searchsorted(pm.embed_rows, [c0, c0 + n])
            h = self.model.forward(seq, ids, positions=torch.from_numpy(pm.positions[c0:c0 + n]),
                                   embed_rows=torch.from_numpy(pm.embed_rows[lo:hi].astype(np.int64) - c0),
                                   embed_vals=lane.visual[lo:hi])
        else:
            h = self.model.forward(seq, ids)
        lane.n_cached += n
        if lane.n_cached < len(lane.tokens):
            return None
        lane.last_token = self._sample(lane, self.model.logits(h[-1:])[0])
        return lane.last_token

    def decode_round(self, lanes: Sequence[Lane]) -> List[int]:
        out = []
        for lane in lanes:
            seq = self._seqs[lane.lane_id]
            lane.tokens.append(lane.last_token)
            pos = torch.tensor([lane.n_cached + lane.rope_delta]) if lane.rope_delta else None
            h = self.model.forward(seq, torch.tensor([lane.last_token]), positions=pos)
            lane.n_cached += 1
            lane.last_token = self._sample(lane, self.model.logits(h)[0])
            out.append(lane.last_token)
        return out


class PackageProgram(ReferenceProgram):
    """CPU program of an attention-only package on its fp32 oracle (models/all_attention.py): the same lanes, sampling,
    frontiers and cold copies as the hybrid oracle program, another decoder underneath."""
    supports_injection = False      # this decoder's forward takes token ids only

    def __init__(self, pkg, weights, max_lanes: int = 8, max_context: int = 4096):
        from ..models.all_attention import PackageReference, PackageSequence, package_model_config
        ProgramBase.__init__(self, package_model_config(pkg, max_context), max_lanes, max_context)
        self.pkg = pkg
        self.model = PackageReference(pkg, weights)
        self._Seq = lambda cfg, fmt: PackageSequence(pkg)
        self.kv_fmt = R.KV_BF16
        self._seqs: Dict[int, object] = {}
        self._slots = 0

