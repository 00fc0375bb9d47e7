"""Native DFlash drafter: context append and one-pass block proposal on the engine's own kernels.

The draft decoder is a `HybridModel` over the weights under `dflash/` (every layer a gated full-attention layer), so
the proposal pass is the target's own step machinery: one ragged step whose chunks are the K-token blocks
`[anchor, MASK, ...]` at each sequence's frontier, with a visibility mask that lets every block position see every
other one (the tree-verify mask with all K bits set) and, on the local layers, a sliding window over the context.
The context append is the only DFlash-specific sequence of launches: feature projection GEMM, RMSNorm, and per draft
layer one K / V projection GEMM whose rows go through the KV quantize-append kernel (key norm, RoPE, page write).
The block's own K / V rows land at the frontier positions and are overwritten by the context rows of the tokens that
get committed there.  Math and oracle: models/dflash.py; reference:
src/targets/qwen3_6/impl/runtime/dflash_impl.h:98-551.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..models.config import ModelConfig
from ..models.dflash import DFlashConfig, draft_model_config
from ..models.hybrid import EPI_STORE, HybridModel, Workspace
from .arena import BumpArena
from .batch import SeqChunk, StepBuffers
from .kv_cache import CyclicKvCache, PagedKvCache


class _SplitKv:
    """The draft decoder's cache as the model sees it: the planes of the sliding-window layers live in a cyclic cache
    (a bounded ring of pages per row) and carry that cache's block table, the other layers live in a full cache."""

    def __init__(self, local: Optional[CyclicKvCache], full: Optional[PagedKvCache]):
        self.local, self.full = local, full
        main = full if full is not None else local
        self.page_size, self.table = main.page_size, main.table
        self.layers = []
        if local is not None:
            for pl in local.layers:
                if full is not None:
                    pl.block_table = local.table
                self.layers.append(pl)
        if full is not None:
            self.layers.extend(full.layers)

    def table_of(self, layer: int) -> torch.Tensor:
        pl = self.layers[layer]
        return pl.block_table if pl.block_table is not None else self.table

    def ensure(self, row: int, n_tokens: int) -> None:
        for c in (self.local, self.full):
            if c is not None:
                c.ensure(row, n_tokens)

    def publish(self) -> None:
        for c in (self.local, self.full):
            if c is not None:
                c.publish()

    def free_row(self, row: int) -> None:
        for c in (self.local, self.full):
            if c is not None:
                c.free_row(row)


class DFlashDrafter:
    def __init__(self, target: ModelConfig, dc: DFlashConfig, weights: Dict[str, torch.Tensor], device, max_batch: int,
                 max_context: int, draft_tokens: int, page_size: int = 64, pdl: bool = False, max_append: int = 2048):
        self.dc = dc.resolved(target)
        self.cfg = cfg = draft_model_config(target, self.dc)
        self.K = K = draft_tokens
        if K < 1 or K > 63:
            raise ValueError("a DFlash block holds 1..63 positions (one visibility bit each)")
        self.device = dev = torch.device(device)
        self.model = HybridModel(cfg, weights, dev, pdl=pdl, prefix="dflash")
        self.model.layer_window = {l: self.dc.window for l in range(self.dc.local_layers)}
        T = max_batch * K
        self.max_append = max(max_append, T)
        self.ws = Workspace(cfg, self.max_append, T, dev)
        ctx = max_context + K + 1
        pages_per_row = (ctx + page_size - 1) // page_size
        n_local, n_full = self.dc.local_layers, cfg.n_layers - self.dc.local_layers
        # the block of K positions is written past the frontier and must stay inside the ring: window + K keys live
        local = CyclicKvCache(cfg, self.dc.window + K, page_size, max_batch, ctx, dev, formats="bf16",
                              n_layers=n_local) if n_local else None
        full = PagedKvCache(cfg, max_batch * pages_per_row, page_size, max_batch, pages_per_row, dev, formats="bf16",
                            n_layers=n_full) if n_full else None
        self.kv = _SplitKv(local, full)
        self.bufs = StepBuffers(T, max_batch, dev, attn_block_tokens=16, max_logit_rows=T)
        # scratch of the context append: the two context copies live for the whole append, the per-layer K / V
        # projection and the append kernel's query output share one scope that every layer reuses
        h, n = cfg.hidden, self.max_append
        self.arena = BumpArena(2 * (2 * n * h + n * 3 * cfg.kv_dim) + 4 * 256, dev)
        self.ctx_raw = self.arena.alloc((n, h), torch.bfloat16, "projected features")
        self.ctx = self.arena.alloc((n, h), torch.bfloat16, "context (normed)")
        with self.arena.scope():
            self.ctx_kv = self.arena.alloc((n, 2 * cfg.kv_dim), torch.bfloat16, "layer context K / V")
            self.q_scratch = self.arena.alloc((n, cfg.kv_dim), torch.bfloat16, "append kernel query scratch")
        self.all_bits = (1 << K) - 1
        self.proposals = 0

    @property
    def n_features(self) -> int:
        return len(self.dc.feature_layers)

    def reset(self, rows: Sequence[int]) -> None:
        for r in rows:
            self.kv.free_row(r)

    # ---- context append ----
    def append_context(self, features: torch.Tensor, table_row: torch.Tensor, positions: torch.Tensor,
                       row_ends: Dict[int, int]) -> None:
        """features [n, F * hidden] bf16 of n committed tokens, their block-table rows and cache positions (int32,
        device); `row_ends`: for every row that appears, one past its largest position (page allocation)."""
        m, cfg, ops = self.model, self.cfg, self.model.ops
        for r, end in row_ends.items():
            self.kv.ensure(r, end + self.K + 1)
        self.kv.publish()
        n_all = features.shape[0]
        for s in range(0, n_all, self.max_append):
            n = min(self.max_append, n_all - s)
            f, rows, pos = features[s:s + n], table_row[s:s + n], positions[s:s + n]
            raw, c = self.ctx_raw[:n], self.ctx[:n]
            m._gemm(f, m.w["dflash/feature_proj"], raw, EPI_STORE)
            m._add_rmsnorm(None, 0, None, raw, None, m.w["dflash/context_norm"], c, n, cfg.hidden)
            for l in range(cfg.n_layers):
                kvp = self.ctx_kv[:n]
                m._gemm(c, m.w[f"dflash/layers/{l}/ctx_kv"], kvp, EPI_STORE)
                planes = self.kv.layers[l]
                kn = m.w[f"dflash/layers/{l}/attn/k_norm"]
                # the append kernel wants query heads as well: the key columns stand in for them (n_q = n_kv), its
                # query output goes to scratch
                ops.attn_prep(kvp, 0, 0, cfg.kv_dim, cfg.n_kv_heads, cfg.n_kv_heads, cfg.head_dim, kn, kn, cfg.rms_eps, True,
                              cfg.rot_dim, m.inv_freq, m.rope_factor, pos, rows, pos, self.kv.table_of(l),
                              self.q_scratch[:n].view(n, cfg.n_kv_heads, cfg.head_dim), planes.k_codes, planes.v_codes,
                              planes.k_scales, planes.v_scales, self.kv.page_size, planes.fmt, planes.group, m.pdl)

    # ---- proposal ----
    def propose(self, rows: Sequence[int], anchors: Sequence[int], frontiers: Sequence[int]) -> torch.Tensor:
        """K draft tokens per sequence ([B, K] int32 on the device): block [anchor, MASK x (K - 1)] at the frontier."""
        B, K, dev = len(rows), self.K, self.device
        for r, n in zip(rows, frontiers):
            self.kv.ensure(r, n + K + 1)
        self.kv.publish()
        chunks = [SeqChunk(rows[b], 0, frontiers[b], [anchors[b]] + [self.dc.mask_token] * (K - 1), True, True)
                  for b in range(B)]
        batch = self.bufs.build(chunks)
        n0 = torch.tensor(list(frontiers), dtype=torch.int32, device=dev)[:, None]
        batch.kv_len.view(B, K).copy_((n0 + K).expand(B, K))          # every block position sees the whole block
        batch.tree_mask = torch.full((B * K,), self.all_bits, dtype=torch.int64, device=dev)
        batch.tree_base = n0.expand(B, K).reshape(-1).contiguous()
        batch.max_kv_len = max(frontiers) + K
        hidden = self.model.forward_hidden(self.ws, batch, self.kv, None)
        lg = self.model.logits(self.ws, batch, hidden)
        ids = self.ws.next_ids[:B * K]
        self.model.ops.argmax_rows(lg, ids, self.model.pdl)
        self.proposals += 1
        return ids.view(B, K)

    def logits(self, rows: Sequence[int], anchors: Sequence[int], frontiers: Sequence[int]) -> torch.Tensor:
        """The proposal pass's logits [B, K, vocab] (tests compare them with the oracle's)."""
        self.propose(rows, anchors, frontiers)
        B = len(rows)
        return self.ws.logits[:B * self.K].view(B, self.K, -1)
