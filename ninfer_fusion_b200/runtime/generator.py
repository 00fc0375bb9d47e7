"""Static-batch generation driver: chunked ragged prefill + CUDA-graph decode.

This is the thin program layer under the engine: it owns the model, the paged
KV cache, the GDN state pool, the workspaces and one captured decode graph per
(batch size, context bucket) -- the counterpart of the reference's graph
families keyed by (B, frontier range) (src/targets/qwen3_6_27b/impl/variant.cpp:190-194,
program_impl.h:17385-17435).  A decode round is: fill the pinned step
descriptor, one H2D copy, one graph launch, one D2H copy of the new token ids.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.hybrid import HybridModel, ShardGeometry, StepBatch, Workspace, pick_attention_split
from .batch import SeqChunk, StepBuffers
from .kv_cache import GdnStatePool, PagedKvCache


def context_bucket(n: int) -> int:
    b = 128
    while b < n:
        b *= 2
    return b


class Generator:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], device, max_batch: int, max_context: int,
                 kv_format: str | Sequence[str] = "bf16", page_size: int = 64, prefill_chunk: int = 2048,
                 use_graph: bool = True, pdl: bool = False, int8_group: int = 64,
                 shard: Optional[ShardGeometry] = None, comm=None, max_logit_rows: int = 0,
                 weight_budget_bytes: Optional[int] = None):
        self.cfg = cfg
        self.device = torch.device(device)
        if weight_budget_bytes is not None:
            # layers beyond the budget live in pinned host memory and rotate through a device arena; the host copies
            # cannot be baked into a decode graph, so such a model runs eagerly
            from .weight_offload import OffloadedWeights
            weights = OffloadedWeights(weights, self.device, int(weight_budget_bytes))
            if weights.plan.offloaded_layers:
                use_graph = False
        self.max_batch, self.max_context = max_batch, max_context
        self.page_size = page_size
        self.prefill_chunk = prefill_chunk
        self.use_graph = use_graph and self.device.type == "cuda"
        self.model = HybridModel(cfg, weights, device, pdl=pdl, shard=shard)
        self.model.comm = comm
        g = self.model.g
        pages_per_row = (max_context + page_size - 1) // page_size
        self.kv = PagedKvCache(cfg, max_batch * pages_per_row, page_size, max_batch, pages_per_row, device,
                               formats=kv_format, int8_group=int8_group, n_kv_heads=g.n_kv_heads)
        self.states = GdnStatePool(cfg, max_batch, device, n_qk_heads=g.gdn_qk_heads, n_v_heads=g.gdn_v_heads)
        cap = max(prefill_chunk, max_batch)
        self.ws = Workspace(cfg, cap, max(max_batch, max_logit_rows), device, shard=shard,
                            x_buffer=None if comm is None else comm.x)
        qt = int(self.model.ops.prefill_attn_block_tokens(g.n_q_heads, g.n_kv_heads)) if self.device.type == "cuda" else 16
        self.bufs_prefill = StepBuffers(cap, max_batch, device, attn_block_tokens=qt)
        self.bufs_decode = StepBuffers(max_batch, max_batch, device, attn_block_tokens=qt)
        pin = self.device.type == "cuda"
        self.out_host = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self._graph_batches: Dict[tuple, StepBatch] = {}
        # per-sequence host state
        self.rows: List[int] = []
        self.slots: List[int] = []
        self.lengths: List[int] = []
        self.last_tokens: List[int] = []
        self.rope_delta: List[int] = []   # per sequence: rope position - cache position after a multimodal prompt
        self.vision = None                # VisionTower, attached by the caller for multimodal prompts
        self._bufs_prefill_mm = None
        self.launches_per_step = 0

    # ------------------------------------------------------------------ sequences
    def reset(self) -> None:
        for r in self.rows:
            self.kv.free_row(r)
        for s in self.slots:
            self.states.release(s)
        self.rows, self.slots, self.lengths, self.last_tokens, self.rope_delta = [], [], [], [], []

    def _encode_media(self, media) -> List[Optional[torch.Tensor]]:
        """Runs the vision tower over every prompt's media; one [V, hidden] tensor per prompt (None = text only)."""
        from ..models.vision import build_control
        if self.vision is None:
            raise ValueError("prompt carries media but no vision tower is attached")
        out: List[Optional[torch.Tensor]] = []
        for pm in media:
            if pm is None or not pm.items:
                out.append(None)
                continue
            control = build_control(pm.grids, self.vision.cfg.merge)
            if control.n_tokens != len(pm.embed_rows):
                raise ValueError("pad-token count does not match the media grids")
            out.append(self.vision.encode(pm.patches(), control))
        return out

    def prefill(self, prompts: Sequence[Sequence[int]], media: Optional[Sequence] = None) -> List[int]:
        """Prefill all prompts (chunked, ragged-packed); returns each sequence's first new token.

        `media[b]` (optional) is the prepared multimodal prompt of sequence b (frontend.media.PreparedPrompt whose
        ids equal prompts[b]): its visual tokens replace the pad-token embeddings and its three-axis positions
        drive the rope; later decode positions are shifted by its rope_delta."""
        if len(prompts) > self.max_batch:
            raise ValueError("too many sequences")
        self.reset()
        B = len(prompts)
        bufs = self.bufs_prefill
        visual: List[Optional[torch.Tensor]] = [None] * B
        if media is not None and any(m is not None for m in media):
            if len(media) != B or any(m is not None and list(m.ids) != list(prompts[b]) for b, m in enumerate(media)):
                raise ValueError("media must hold one prepared prompt (or None) per sequence, with the same ids")
            visual = self._encode_media(media)
            if self._bufs_prefill_mm is None:
                self._bufs_prefill_mm = StepBuffers(bufs.max_tokens, bufs.max_seqs, self.device, mrope=True,
                                                    attn_block_tokens=bufs.attn_block_tokens)
            bufs = self._bufs_prefill_mm
        self.rope_delta = [0 if (media is None or media[b] is None) else int(media[b].rope_delta) for b in range(B)]
        for b in range(B):
            self.rows.append(b)
            self.slots.append(self.states.alloc())
            self.lengths.append(0)
            self.kv.ensure(b, len(prompts[b]) + 1)
        self.kv.publish()
        first = [0] * B
        cursor = [0] * B
        pending = list(range(B))
        while pending:
            budget = self.prefill_chunk
            chunks, owners = [], []
            e_rows, e_vals = [], []
            for b in list(pending):
                if budget == 0 or len(chunks) == self.max_batch:
                    break
                n = min(budget, len(prompts[b]) - cursor[b])
                done = cursor[b] + n == len(prompts[b])
                chunk = SeqChunk(self.rows[b], self.slots[b], cursor[b], prompts[b][cursor[b]:cursor[b] + n], done)
                if visual[b] is not None:
                    pm = media[b]
                    chunk.positions = pm.positions[cursor[b]:cursor[b] + n]
                    lo, hi = np.searchsorted(pm.embed_rows, [cursor[b], cursor[b] + n])
                    if hi > lo:
                        step_row0 = self.prefill_chunk - budget
                        e_rows.append(torch.from_numpy(pm.embed_rows[lo:hi].astype(np.int64) - cursor[b] + step_row0))
                        e_vals.append(visual[b][lo:hi])
                chunks.append(chunk)
                owners.append((b, done))
                cursor[b] += n
                budget -= n
                if done:
                    pending.remove(b)
            batch = bufs.build(chunks)
            if e_rows:
                batch.embed_rows = torch.cat(e_rows).to(self.device, non_blocking=True)
                batch.embed_vals = torch.cat(e_vals)
            ids = self.model.forward_greedy(self.ws, batch, self.kv, self.states)
            if ids.numel():
                self.out_host[: ids.numel()].copy_(ids, non_blocking=True)
                torch.cuda.current_stream().synchronize() if self.device.type == "cuda" else None
                j = 0
                for b, done in owners:
                    if done:
                        first[b] = int(self.out_host[j])
                        j += 1
        for b in range(B):
            self.lengths[b] = len(prompts[b])
        self.last_tokens = list(first)
        self.model.status.check("after prefill")
        return first

    # ------------------------------------------------------------------ decode
    def _decode_chunks(self) -> List[SeqChunk]:
        return [SeqChunk(self.rows[b], self.slots[b], self.lengths[b], [self.last_tokens[b]], True)
                for b in range(len(self.rows))]

    def _ensure_pages(self, extra: int = 1) -> None:
        for b, r in enumerate(self.rows):
            self.kv.ensure(r, self.lengths[b] + extra)
        self.kv.publish()

    def _graph_for(self, B: int, bucket: int, advance: bool):
        key = (B, bucket, advance)
        if key in self._graphs:
            return self._graphs[key], self._graph_batches[key]
        batch = self.bufs_decode.build(self._decode_chunks(), upload=True, rope_delta=self.rope_delta)
        batch.max_kv_len = bucket  # bake the bucket's split geometry, not this step's
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up outside capture (sets kernel attributes, fills caches)
                self._snapshot_states()
                self.model.forward_greedy(self.ws, batch, self.kv, self.states)
                self._rollback_states()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        self._snapshot_states()
        with torch.cuda.graph(graph):
            ids = self.model.forward_greedy(self.ws, batch, self.kv, self.states)
            if advance:
                batch.ids.copy_(ids)
                batch.cache_pos.add_(1)
                batch.kv_len.add_(1)
                batch.rope_pos.add_(1)
        self._rollback_states()
        self._graphs[key] = graph
        self._graph_batches[key] = batch
        return graph, batch

    def _snapshot_states(self) -> None:
        """Warm-up / capture runs must not advance the recurrent state."""
        self._saved = [(c.clone(), s.clone()) for c, s in zip(self.states.conv, self.states.ssm)]

    def _rollback_states(self) -> None:
        torch.cuda.synchronize(self.device)
        for (c0, s0), c, s in zip(self._saved, self.states.conv, self.states.ssm):
            c.copy_(c0)
            s.copy_(s0)
        self._saved = None

    def decode_step(self) -> List[int]:
        """One decode round through the public path: H2D descriptors, graph (or eager), D2H ids."""
        B = len(self.rows)
        self._ensure_pages(1)
        if self.use_graph:
            bucket = context_bucket(max(self.lengths) + 1)
            graph, _ = self._graph_for(B, bucket, advance=False)
            self.bufs_decode.build(self._decode_chunks(), upload=True, rope_delta=self.rope_delta)
            graph.replay()
            ids = self.ws.next_ids[:B]
        else:
            batch = self.bufs_decode.build(self._decode_chunks(), upload=True, rope_delta=self.rope_delta)
            ids = self.model.forward_greedy(self.ws, batch, self.kv, self.states)
        self.out_host[:B].copy_(ids, non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        toks = [int(v) for v in self.out_host[:B]]
        for b in range(B):
            self.lengths[b] += 1
        self.last_tokens = toks
        return toks

    def decode_device_loop(self, n_steps: int):
        """n_steps decode rounds with no host round trip (token ids and positions advance on the
        device inside the graph).  Used for device-side timing; returns the graph and a
        finaliser that brings the host state up to date."""
        B = len(self.rows)
        self._ensure_pages(n_steps + 1)
        bucket = context_bucket(max(self.lengths) + n_steps + 1)
        graph, batch = self._graph_for(B, bucket, advance=True)
        self.bufs_decode.build(self._decode_chunks(), upload=True, rope_delta=self.rope_delta)

        def finish():
            self.out_host[:B].copy_(self.ws.next_ids[:B])
            torch.cuda.synchronize(self.device)
            for b in range(B):
                self.lengths[b] += n_steps
            self.last_tokens = [int(v) for v in self.out_host[:B]]

        return graph, finish

    def generate(self, prompts: Sequence[Sequence[int]], n_new: int) -> List[List[int]]:
        first = self.prefill(prompts)
        out = [[t] for t in first]
        for _ in range(n_new - 1):
            toks = self.decode_step()
            for b, t in enumerate(toks):
                out[b].append(t)
        self.model.status.check("after decode")
        return out
