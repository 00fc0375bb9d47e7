"""GPU program: lanes on the native kernels, CUDA graph per (batch size, context bucket, sampler kind).

Decode round = fill the pinned step descriptor (+ per-row sampling parameters), one H2D copy, one graph
launch (forward + arg-max or sampler + penalty-count update), one D2H copy of the token ids.  Prefill
advances one lane by a chunk through the same ragged forward.  See `program.ProgramBase` for the verbs.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..utils import trace

from ..models.config import ModelConfig
from ..models.hybrid import HybridModel, ShardGeometry, StepBatch, Workspace
from .batch import SeqChunk, StepBuffers
from .generator import context_bucket
from .kv_cache import GdnStatePool, PagedKvCache
from .program import Lane, ProgramBase, SamplingParams


class GpuProgram(ProgramBase):
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], device, max_lanes: int = 32,
                 max_context: int = 8192, kv_format="bf16", page_size: int = 64, prefill_chunk: int = 2048,
                 use_graph: bool = True, pdl: bool = True, int8_group: int = 64, kv_pages: Optional[int] = None,
                 shard: Optional[ShardGeometry] = None, comm=None, penalties: bool = False,
                 checkpoint_slots: Optional[int] = None, weight_budget_bytes: Optional[int] = None,
                 mixed_capacity: Optional[Sequence[int]] = None, mixed_hot_tier: int = 0, descent=None):
        """`kv_format` "mixed" (or a per-layer list with "mixed" entries): those layers keep their cells in three
        precision tiers; `mixed_capacity` = cells per tier and layer, `descent` = a kv.descent.DescentConfig that
        `kv_descent_step` applies between rounds (None = cells only move when `kv.descend` is called by hand)."""
        super().__init__(cfg, max_lanes, max_context)
        if weight_budget_bytes is not None:
            from .weight_offload import OffloadedWeights
            weights = OffloadedWeights(weights, device, int(weight_budget_bytes))
            if weights.plan.offloaded_layers:
                use_graph = False   # host copies cannot be baked into a decode graph
        # recurrent-state slots beyond the lanes hold the state images of session checkpoints (the reference keeps 2C)
        self.checkpoint_slots = max_lanes if checkpoint_slots is None else checkpoint_slots
        self.max_checkpoints = self.checkpoint_slots
        self.device = torch.device(device)
        self.prefill_chunk = prefill_chunk
        self.use_graph = use_graph
        self.model = HybridModel(cfg, weights, device, pdl=pdl, shard=shard)
        self.model.comm = comm
        g = self.model.g
        pages_per_row = (max_context + page_size - 1) // page_size
        n_pages = kv_pages if kv_pages is not None else max_lanes * pages_per_row
        self.kv = PagedKvCache(cfg, n_pages, page_size, max_lanes, pages_per_row, device, formats=kv_format,
                               int8_group=int8_group, n_kv_heads=g.n_kv_heads, mixed_capacity=mixed_capacity,
                               mixed_hot_tier=mixed_hot_tier)
        self.descent = descent
        self.descent_stats = {"passes": 0, "cells_moved": 0}
        self.states = GdnStatePool(cfg, max_lanes + self.checkpoint_slots, device, n_qk_heads=g.gdn_qk_heads,
                                   n_v_heads=g.gdn_v_heads)
        self._ckpt_slots_free = self.checkpoint_slots
        cap = max(prefill_chunk, max_lanes)
        self.ws = Workspace(cfg, cap, max_lanes, device, shard=shard, x_buffer=None if comm is None else comm.x)
        qt = int(self.model.ops.prefill_attn_block_tokens(g.n_q_heads, g.n_kv_heads))
        self.bufs_prefill = StepBuffers(cap, max_lanes, device, attn_block_tokens=qt)
        self.bufs_decode = StepBuffers(max_lanes, max_lanes, device, attn_block_tokens=qt)
        self.out_host = torch.zeros(max_lanes, dtype=torch.int32, pin_memory=True)
        # per-row sampling parameters (pinned host + device twins), filled every sampled round
        B = max_lanes
        self.sp_host = {"temperature": torch.zeros(B, pin_memory=True), "top_p": torch.ones(B, pin_memory=True),
                        "min_p": torch.zeros(B, pin_memory=True), "presence": torch.zeros(B, pin_memory=True),
                        "frequency": torch.zeros(B, pin_memory=True),
                        "top_k": torch.zeros(B, dtype=torch.int32, pin_memory=True),
                        "seeds": torch.zeros(B, dtype=torch.int64, pin_memory=True),
                        "positions": torch.zeros(B, dtype=torch.int32, pin_memory=True)}
        self.sp_dev = {k: v.to(self.device) for k, v in self.sp_host.items()}
        self.penalties = penalties
        self.token_counts = (torch.zeros((B, g.vocab_rows), dtype=torch.int32, device=self.device)
                             if penalties and comm is None else None)
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.vision = None
        self._bufs_prefill_mm = None

    # ------------------------------------------------------------------ lanes
    def _alloc_slot(self) -> int:
        return self.states.alloc()

    def _release(self, lane: Lane) -> None:
        self.kv.free_row(lane.row)
        self.states.release(lane.slot)
        if self.token_counts is not None:
            self.token_counts[lane.row].zero_()

    # ------------------------------------------------------------------ session checkpoints
    def _snapshot(self, lane: Lane, n_tokens: int):
        if self._ckpt_slots_free <= 0:
            return None
        pages = self.kv.detach_prefix(lane.row, n_tokens)
        if pages is None:
            return None
        self._ckpt_slots_free -= 1
        slot = self.states.alloc()
        self.states.copy_slot(lane.slot, slot)
        return (pages, slot)

    def _restore(self, handle, lane: Lane, n_tokens: int) -> None:
        pages, slot = handle
        self.kv.attach_prefix(pages, lane.row, n_tokens)
        self.states.copy_slot(slot, lane.slot)

    def _drop(self, handle) -> None:
        pages, slot = handle
        self.kv.drop_pages(pages)
        self.states.release(slot)
        self._ckpt_slots_free += 1

    def _demote(self, handle):
        """Device frontier -> pinned host copy (KV pages of every layer + the state image)."""
        pages, slot = handle
        return {"n_pages": len(pages), "tensors": [self.kv.export_pages(pages), self.states.export_slot(slot)]}

    def _promote(self, cold):
        if self._ckpt_slots_free <= 0:
            return None
        pages = self.kv.import_pages(cold["tensors"][0], cold["n_pages"])
        if pages is None:
            return None
        self._ckpt_slots_free -= 1
        slot = self.states.alloc()
        self.states.import_slot(cold["tensors"][1], slot)
        return (pages, slot)

    def set_global_tokens(self, n_tokens: int) -> None:
        """Expert parallelism: bound on the tokens that all ranks together run in the next step (the MoE exchange
        sizes its tiles and receive rows by it)."""
        self.model.moe_global_tokens = int(n_tokens)

    def _wait_device(self) -> None:
        """Blocks until the step's results are on the host; the blocked time is the step's exposed device wait."""
        t0 = time.perf_counter()
        torch.cuda.current_stream().synchronize()
        self.device_wait_s += time.perf_counter() - t0

    def _pages_for(self, n_tokens: int) -> int:
        return (max(0, n_tokens) + self.kv.page_size - 1) // self.kv.page_size

    def _pages_free(self) -> int:
        return int(self.kv.pool.free_pages)

    def _pages_held(self, lane: Lane) -> int:
        return len(self.kv.row_pages.get(lane.row, ()))

    def _kv_room(self, n_tokens: int) -> bool:
        need = self._pages_for(n_tokens)
        if self.pages_available() < need:   # free pages minus what admitted requests may still take
            return False
        # mixed layers: every new page needs a cell in the hot tier of each of them
        return all(len(l.free[l.hot_tier]) >= need for l in self.kv.mixed)

    # ------------------------------------------------------------------ per-cell precision descent
    def kv_descent_step(self) -> int:
        """One descent pass over the live lanes' cells (kv/descent.py decides which, one rung per cell and pass,
        oldest first, under the configured budgets); the re-encoding runs on the device.  Called by the engine
        between rounds.  Returns the number of cells moved."""
        if self.descent is None or not self.kv.mixed or not self.lanes:
            return 0
        from ..kv.descent import CellMap, plan_descent_pass
        mixed_idx = [i for i, l in enumerate(self.kv.layers) if l in self.kv.mixed]
        cells = CellMap(self.kv.page_size, len(mixed_idx))
        page_of = {}
        for lane in self.lanes.values():
            pages = self.kv.row_pages.get(lane.row, [])
            cells.frontier[lane.lane_id] = lane.n_cached
            for b, pg in enumerate(pages[: (lane.n_cached + self.kv.page_size - 1) // self.kv.page_size]):
                if pg < 0:
                    continue
                for j, li in enumerate(mixed_idx):
                    t = self.kv.layers[li].tier_of(pg)
                    if t >= 0:
                        cells.rungs[(lane.lane_id, j, b)] = t
                        page_of[(lane.lane_id, j, b)] = pg
        moves = plan_descent_pass(cells, self.descent, self.model.g.n_kv_heads, self.cfg.head_dim)
        by_target: Dict[tuple, List[int]] = {}
        for m in moves:
            if m.dst == "cold":
                continue
            by_target.setdefault((mixed_idx[m.layer], self.descent.ladder.index(m.dst)), []).append(page_of[(m.seq, m.layer, m.block)])
        moved = 0
        for (li, tier), pages in by_target.items():
            moved += self.kv.descend(li, sorted(set(pages)), tier)
        if moved:
            self.descent_stats["passes"] += 1
            self.descent_stats["cells_moved"] += moved
        return moved

    def census(self) -> dict:
        c = super().census()
        if self.kv.mixed:
            c["kv_tiers"] = self.kv.tier_census()
            c["kv_bytes_in_use"] = self.kv.bytes_in_use()
            c["kv_descent"] = dict(self.descent_stats)
        return c

    # ------------------------------------------------------------------ sampling
    def _fill_sampling(self, lanes: Sequence[Lane]) -> bool:
        """Returns True when every lane is greedy (arg-max graph)."""
        if all(l.sampling.greedy for l in lanes):
            return True
        h = self.sp_host
        for i, l in enumerate(lanes):
            s = l.sampling
            h["temperature"][i] = s.temperature
            h["top_k"][i] = s.top_k
            h["top_p"][i] = s.top_p
            h["min_p"][i] = s.min_p
            h["presence"][i] = s.presence_penalty
            h["frequency"][i] = s.frequency_penalty
            h["seeds"][i] = s.seed
            h["positions"][i] = len(l.tokens)
        for k in h:
            self.sp_dev[k].copy_(h[k], non_blocking=True)
        return False

    def _select(self, logits: torch.Tensor, rows: torch.Tensor, greedy: bool, out: torch.Tensor) -> None:
        ops = self.model.ops
        n = logits.shape[0]
        if greedy:
            if self.model.comm is not None:
                self.model.comm.argmax(self.model, logits, out)
            else:
                ops.argmax_rows(logits, out, self.model.pdl)
            return
        if self.model.comm is not None:
            raise NotImplementedError("stochastic sampling under tensor parallelism needs gathered logits")
        d = self.sp_dev
        counts = None
        if self.token_counts is not None:
            counts = self.token_counts.index_select(0, rows.long())
        ops.sample_rows(logits, d["temperature"][:n], d["top_k"][:n], d["top_p"][:n], d["min_p"][:n],
                        d["presence"][:n] if counts is not None else None,
                        d["frequency"][:n] if counts is not None else None, counts, d["seeds"][:n],
                        d["positions"][:n], 0, out, None)

    def _forward_select(self, batch: StepBatch, greedy: bool, rows: torch.Tensor) -> torch.Tensor:
        hidden = self.model.forward_hidden(self.ws, batch, self.kv, self.states)
        if batch.logit_rows.numel() == 0:
            return self.ws.next_ids[:0]
        lg = self.model.logits(self.ws, batch, hidden)
        out = self.ws.next_ids[: lg.shape[0]]
        self._select(lg, rows, greedy, out)
        return out

    # ------------------------------------------------------------------ prefill
    def prefill_step(self, lane: Lane, budget: int) -> Optional[int]:
        n = min(budget, self.prefill_chunk, len(lane.tokens) - lane.n_cached)
        done = lane.n_cached + n == len(lane.tokens)
        self.kv.ensure(lane.row, lane.n_cached + n + 1)
        self.kv.publish()
        chunk = SeqChunk(lane.row, lane.slot, lane.n_cached, lane.tokens[lane.n_cached:lane.n_cached + n], done)
        if lane.media is not None:
            batch = self._build_media_chunk(lane, chunk, n)
        else:
            batch = self.bufs_prefill.build([chunk])
        greedy = self._fill_sampling([lane]) if done else True
        rows = torch.tensor([lane.row], device=self.device)
        ids = self._forward_select(batch, greedy, rows)
        lane.n_cached += n
        if not done:
            return None
        self.out_host[:1].copy_(ids[:1], non_blocking=True)
        self._wait_device()
        self.model.status.check("after prefill")
        lane.last_token = int(self.out_host[0])
        return lane.last_token

    def attach_vision(self, tower) -> None:
        """Enables multimodal requests: `tower` is a models.vision.VisionTower whose output width is the text hidden."""
        if tower.cfg.out_hidden != self.cfg.hidden:
            raise ValueError("vision tower output width differs from the text hidden size")
        self.vision = tower
        self.supports_media = True

    def _build_media_chunk(self, lane: Lane, chunk: SeqChunk, n: int) -> StepBatch:
        """Step descriptor of a multimodal prompt chunk: three-axis positions, visual rows over the pad embeddings."""
        from ..models.vision import build_control
        pm = lane.media
        if lane.visual is None:
            control = build_control(pm.grids, self.vision.cfg.merge)
            if control.n_tokens != len(pm.embed_rows):
                raise ValueError("pad-token count does not match the media grids")
            lane.visual = self.vision.encode(pm.patches(), control)
        if self._bufs_prefill_mm is None:
            b = self.bufs_prefill
            self._bufs_prefill_mm = StepBuffers(b.max_tokens, b.max_seqs, self.device, mrope=True,
                                                attn_block_tokens=b.attn_block_tokens)
        c0 = lane.n_cached
        chunk.positions = pm.positions[c0:c0 + n]
        batch = self._bufs_prefill_mm.build([chunk])
        lo, hi = np.searchsorted(pm.embed_rows, [c0, c0 + n])
        if hi > lo:
            batch.embed_rows = torch.from_numpy(pm.embed_rows[lo:hi].astype(np.int64) - c0).to(self.device, non_blocking=True)
            batch.embed_vals = lane.visual[lo:hi]
        if c0 + n == len(lane.tokens):
            lane.visual = None   # the tower's output is not needed after the prompt
        return batch

    # ------------------------------------------------------------------ decode
    def _chunks(self, lanes: Sequence[Lane]) -> List[SeqChunk]:
        return [SeqChunk(l.row, l.slot, l.n_cached, [l.last_token], True) for l in lanes]

    def _graph_for(self, lanes: Sequence[Lane], bucket: int, greedy: bool) -> torch.cuda.CUDAGraph:
        key = (len(lanes), bucket, greedy)
        g = self._graphs.get(key)
        if g is not None:
            return g
        batch = self.bufs_decode.build(self._chunks(lanes), upload=True, rope_delta=[l.rope_delta for l in lanes])
        batch.max_kv_len = bucket
        rows = batch.table_row
        saved = [(c.clone(), s.clone()) for c, s in zip(self.states.conv, self.states.ssm)]
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                self._forward_select(batch, greedy, rows)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._forward_select(batch, greedy, rows)
        torch.cuda.synchronize(self.device)
        for (c0, s0), c, s in zip(saved, self.states.conv, self.states.ssm):
            c.copy_(c0)
            s.copy_(s0)
        self._graphs[key] = g
        return g

    def decode_round(self, lanes: Sequence[Lane]) -> List[int]:
        B = len(lanes)
        if B == 0:
            return []
        for l in lanes:
            l.tokens.append(l.last_token)
            self.kv.ensure(l.row, l.n_cached + 2)
        self.kv.publish()
        greedy = self._fill_sampling(lanes)
        if self.use_graph:
            bucket = context_bucket(max(l.n_cached for l in lanes) + 1)
            graph = self._graph_for(lanes, bucket, greedy)
            self.bufs_decode.build(self._chunks(lanes), upload=True, rope_delta=[l.rope_delta for l in lanes])
            with trace.span("graph", "replay", lanes=B):
                graph.replay()
            ids = self.ws.next_ids[:B]
        else:
            batch = self.bufs_decode.build(self._chunks(lanes), upload=True, rope_delta=[l.rope_delta for l in lanes])
            ids = self._forward_select(batch, greedy, batch.table_row)
        self.out_host[:B].copy_(ids, non_blocking=True)
        self._wait_device()
        toks = [int(v) for v in self.out_host[:B]]
        if self.token_counts is not None:
            r = torch.tensor([l.row for l in lanes], device=self.device)
            self.token_counts[r, torch.tensor(toks, device=self.device)] += 1
        for l, t in zip(lanes, toks):
            l.n_cached += 1
            l.last_token = t
        return toks
