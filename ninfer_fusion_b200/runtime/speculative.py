"""Draft-and-verify speculative decoding: MTP draft module (or a host n-gram drafter), chain verify in
one target pass, greedy acceptance on the device, and replay of the accepted prefix into the GDN state.

One round for every sequence (frontier n = tokens in the target's KV cache, t = last sampled token):

  1. draft      d_1 is already known from the previous round's catch-up; K - 1 single-token steps of
                the draft module (its own hidden state fed back) give d_2..d_K
  2. verify     the target runs [t, d_1..d_K] at positions n..n+K in ONE ragged pass; full-attention
                layers append K/V for all K + 1 positions (rejected ones are simply overwritten later),
                GDN layers leave their state untouched and record their projections
  3. accept     longest prefix with d_{j+1} == argmax_j, plus the target's own next token
  4. fold       the accepted m + 1 tokens are replayed into conv history + recurrent state
  5. catch-up   the draft module re-reads the accepted positions with the TARGET's hidden states
                (overwriting its speculative K/V there) and predicts the next d_1

Reference: src/targets/qwen3_6/impl/runtime/mtp_impl.h, speculative_target_impl.h,
include/ninfer/ops/speculative_round.h:40-151, include/ninfer/ops/gdn_replay.h:13-49
(replay-record + fold), include/ninfer/ops/suffix_lookup.h (n-gram lookup drafts).
"""
from __future__ import annotations

import os
import time
from dataclasses import replace
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..models.config import ModelConfig
from ..models.hybrid import GdnRecords
from .batch import SeqChunk, StepBuffers
from .generator import Generator, context_bucket
from .lookup_fuse import lookup_drafter
from .kv_cache import PagedKvCache


def ngram_drafter(history: Sequence[int], k: int, max_n: int = 4) -> Optional[List[int]]:
    """Suffix lookup: find the most recent earlier occurrence of the longest suffix (up to `max_n` tokens) of
    `history` and propose the k tokens that followed it.  Returns None when nothing matches."""
    L = len(history)
    for n in range(min(max_n, L - 1), 0, -1):
        suffix = list(history[L - n:])
        for start in range(L - n - 1, -1, -1):
            if list(history[start:start + n]) == suffix:
                cont = list(history[start + n:start + n + k])
                if cont:
                    return cont + [cont[-1]] * (k - len(cont))
    return None


class SpeculativeGenerator(Generator):
    """Static-batch greedy generation with K chained draft tokens per round."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], device, max_batch: int, max_context: int,
                 draft_tokens: int = 3, drafter: str = "mtp", sampling=None, tree_ranks: int = 1,
                 stochastic_drafts: bool = False, adaptive_width=False, draft_head_ids=None, **kw):
        K = draft_tokens
        if K < 1:
            raise ValueError("draft_tokens must be >= 1")
        kw.setdefault("use_graph", False)
        dflash_config = kw.pop("dflash_config", None)
        R_ = max(1, tree_ranks)
        if 1 + R_ * K > 64:
            raise ValueError("a verify window holds at most 64 nodes (one visibility bit each)")
        super().__init__(cfg, weights, device, max_batch, max_context, max_logit_rows=max_batch * (1 + R_ * K), **kw)
        self.K = K
        self.R = R_   # candidates per depth of the draft tree: rank 0 extends the chain, ranks 1.. are side branches
        self.sampling = sampling  # runtime.program.SamplingParams for stochastic verification; None / greedy = arg-max
        self.drafter = drafter  # "mtp" | "dflash" | "ngram" | "lookup" | "hook"
        self.draft_hook: Optional[Callable[[int, List[int], int], Optional[List[int]]]] = None
        dev, g = self.device, self.model.g
        Tv = max_batch * (1 + self.R * K)
        qt = self.bufs_decode.attn_block_tokens
        self.bufs_verify = StepBuffers(Tv, max_batch, dev, attn_block_tokens=qt, max_logit_rows=Tv)
        self.bufs_catch = StepBuffers(Tv, max_batch, dev, attn_block_tokens=qt)
        self.bufs_draft = StepBuffers(max_batch, max_batch, dev, attn_block_tokens=qt)
        self.rec = GdnRecords(cfg, Tv, dev, shard=self.model.g)
        h = cfg.hidden
        self.h_keep = torch.empty((max(self.ws.max_tokens, Tv), h), dtype=torch.bfloat16, device=dev)
        self.h_in = torch.empty((max(self.ws.max_tokens, Tv), h), dtype=torch.bfloat16, device=dev)
        self.mtp_h = torch.empty((max_batch, h), dtype=torch.bfloat16, device=dev)
        pin = dev.type == "cuda"
        self.next_host = torch.zeros(max(self.ws.max_tokens, Tv), dtype=torch.int32, pin_memory=pin)
        self.next_dev = torch.zeros(max(self.ws.max_tokens, Tv), dtype=torch.int32, device=dev)
        self.drafts = torch.zeros((max_batch, K), dtype=torch.int32, device=dev)
        self.drafts_r = torch.zeros((max_batch, K, self.R), dtype=torch.int32, device=dev)   # [b, depth, rank]
        self.tree_hook: Optional[Callable[[int, List[int], int, int], Optional[List[List[int]]]]] = None
        self.draft_host = torch.zeros((max_batch, K), dtype=torch.int32, pin_memory=pin)
        self.n_acc = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.out_tok = torch.zeros((max_batch, K + 1), dtype=torch.int32, device=dev)
        self.acc_host = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        self.tok_host = torch.zeros((max_batch, K + 1), dtype=torch.int32, pin_memory=pin)
        # Stochastic drafts (chain mode, MTP drafter, sampled requests): the draft module SAMPLES its proposals from
        # its own processed distribution q and hands q to the verifier, which accepts with min(1, p / q) and resamples
        # a rejection from max(p - q, 0): speculative sampling in its general form.  Off: proposals are arg-max tokens
        # verified with q = 1 at the draft.  Either way the emitted tokens are distributed as the target's p.
        self.stochastic_drafts = bool(stochastic_drafts) and drafter == "mtp" and self.R == 1
        DK = 32   # pairs per exported distribution: the sampler keeps at most its top-k cap (32) candidates
        self.q_ids = torch.full((max_batch, K + 1, DK), -1, dtype=torch.int32, device=dev)
        self.q_probs = torch.zeros((max_batch, K + 1, DK), dtype=torch.float32, device=dev)
        # Adaptive draft width (chained rounds only): one set of [batch, k] buffers and one round graph per ladder
        # width; the first draft of the next round is carried across a change of width.
        self.width_ctl = None
        self._width_bufs = {K: (self.drafts, self.out_tok, self.tok_host, self.draft_host)}
        if adaptive_width:
            if self.R > 1 or self.stochastic_drafts or drafter == "dflash":
                raise ValueError("adaptive width drives chained rounds of the MTP, hook and n-gram drafters")
            from .spec_width import AdaptiveWidth
            self.width_ctl = adaptive_width if isinstance(adaptive_width, AdaptiveWidth) else AdaptiveWidth(max_width=K)
            if self.width_ctl.max_width != K:
                raise ValueError("the width controller's maximum must equal draft_tokens")
        # Shortlist draft head: the draft module's proposals are the arg-max over a subset of the vocabulary (rows of
        # the LM head gathered once), mapped back to token ids.  A draft only has to be right often, not always: the
        # target verifies with the full head, and a draft pass no longer streams the whole LM head.
        self.head_ids = self.head_w = self.head_logits = None
        if draft_head_ids is not None:
            if drafter != "mtp" or self.R > 1 or self.stochastic_drafts:
                raise ValueError("the shortlist head serves chained arg-max drafts of the draft module (no tree ranks, "
                                 "no sampled drafts: both need the full distribution)")
            head = weights[f"{self.model.prefix}/lm_head"]
            if not isinstance(head, torch.Tensor) or head.dtype != torch.bfloat16:
                raise ValueError("the shortlist head is gathered from a bf16 LM head")
            ids = torch.as_tensor(draft_head_ids, dtype=torch.int64).flatten().unique(sorted=True)
            if ids.numel() < 8 or ids.numel() % 8 or int(ids[0]) < 0 or int(ids[-1]) >= head.shape[0]:
                raise ValueError("draft_head_ids: a multiple of 8 distinct token ids inside the vocabulary")
            self.head_ids = ids.to(device=dev, dtype=torch.int32)
            self.head_w = head.index_select(0, ids.to(dev)).contiguous()
            self.head_logits = torch.empty((max(self.ws.max_tokens, Tv), ids.numel()), dtype=torch.bfloat16, device=dev)
        self.kv_mtp = None
        if drafter == "mtp":
            if "mtp/fc" not in weights:
                raise ValueError("weights have no draft module (random_weights(..., with_mtp=True))")
            pages_per_row = (max_context + self.page_size - 1) // self.page_size
            one_attn = cfg.shrink(cfg.full_attn_interval)  # geometry of a cache with a single attention layer
            self.kv_mtp = PagedKvCache(one_attn, max_batch * pages_per_row, self.page_size, max_batch, pages_per_row,
                                       dev, formats="bf16", n_kv_heads=g.n_kv_heads)
        self.dflash = None
        if drafter == "dflash":
            # block-diffusion drafter: conditions on tapped residual streams of the target, proposes K tokens in one pass
            if "dflash/feature_proj" not in weights:
                raise ValueError("weights have no DFlash draft model (models.dflash.random_dflash_weights)")
            if self.R > 1:
                raise ValueError("the DFlash drafter proposes a chain (tree_ranks = 1)")
            from ..models.dflash import DFlashConfig
            from .dflash import DFlashDrafter
            dc = dflash_config or DFlashConfig()
            self.dflash = DFlashDrafter(cfg, dc, weights, dev, max_batch, max_context, K, page_size=self.page_size,
                                        pdl=self.model.pdl, max_append=max(self.ws.max_tokens, Tv))
            fl = self.dflash.dc.feature_layers
            self.model.feature_taps = {layer: i for i, layer in enumerate(fl)}
            self.model.feature_buf = torch.empty((max(self.ws.max_tokens, Tv), len(fl) * h), dtype=torch.bfloat16, device=dev)
        # a chained greedy round as ONE CUDA graph per (batch, context bucket): draft passes, verify, acceptance, state
        # fold and draft catch-up run back to back with the accepted lengths staying on the device
        self.seq_end = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.catch_rows = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.draft_col = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self._round_graphs: Dict[tuple, tuple] = {}
        self.device_wait_s = 0.0
        self.history: List[List[int]] = []
        self.rounds = 0
        self.accepted = 0
        self.emitted = 0

    # ------------------------------------------------------------------ helpers
    def _upload_next(self, toks: Sequence[int]) -> torch.Tensor:
        n = len(toks)
        self.next_host[:n] = torch.tensor(list(toks), dtype=torch.int32)
        self.next_dev[:n].copy_(self.next_host[:n], non_blocking=True)
        return self.next_dev[:n]

    def _sampling_of(self, b: int):
        sp = self.sampling[b] if isinstance(self.sampling, (list, tuple)) else self.sampling
        return sp

    def _draft_stochastically(self) -> bool:
        if not self.stochastic_drafts or self.sampling is None:
            return False
        sps = self.sampling if isinstance(self.sampling, (list, tuple)) else [self.sampling]
        return any(sp is not None and not sp.greedy for sp in sps)

    def _sample_draft(self, lg: torch.Tensor, ids: torch.Tensor, seqs: Sequence[int], col: int) -> None:
        """Draws draft column `col` of the sequences `seqs` (one logit row each, in order) from the draft module's
        distribution under each sequence's own sampling parameters and keeps that distribution as q.  Random stream
        3, so that the proposals are independent of the verifier's accept / resample draws (streams 1 and 2)."""
        dev, n = self.device, len(seqs)

        def rows(get, dtype):
            return torch.tensor([get(self._sampling_of(b)) for b in seqs], dtype=dtype, device=dev)
        pos = torch.tensor([self.lengths[b] + col + 1 for b in seqs], dtype=torch.int32, device=dev)
        q_i = torch.empty((n, self.q_ids.shape[2]), dtype=torch.int32, device=dev)
        q_p = torch.empty((n, self.q_ids.shape[2]), dtype=torch.float32, device=dev)
        q_i.fill_(-1); q_p.zero_()
        self.model.ops.sample_rows(lg, rows(lambda sp: 0.0 if sp is None else sp.temperature, torch.float32),
                                   rows(lambda sp: 1 if sp is None else sp.top_k, torch.int32),
                                   rows(lambda sp: 1.0 if sp is None else sp.top_p, torch.float32),
                                   rows(lambda sp: 0.0 if sp is None else sp.min_p, torch.float32), None, None, None,
                                   rows(lambda sp: 0 if sp is None else sp.seed, torch.int64), pos, 3, ids, None,
                                   None, None, None, None, q_i, q_p)
        # a greedy sequence proposes its arg-max: q is one at that token (the sampler writes no distribution for it)
        greedy = torch.tensor([self._sampling_of(b) is None or self._sampling_of(b).greedy for b in seqs], device=dev)
        if bool(greedy.any()):
            q_i[:, 0] = torch.where(greedy, ids[:n], q_i[:, 0])
            q_p[:, 0] = torch.where(greedy, torch.ones_like(q_p[:, 0]), q_p[:, 0])
        idx = torch.tensor(list(seqs), dtype=torch.long, device=dev)
        self.q_ids[idx, col] = q_i
        self.q_probs[idx, col] = q_p

    def _propose(self, batch, hid: torch.Tensor) -> torch.Tensor:
        """Arg-max proposals of the draft module for the logit rows of `batch` (ws.next_ids[:R]): over the whole
        vocabulary, or over the shortlist head with its ids mapped back (ascending ids, so ties resolve to the
        lowest token id as in the full head)."""
        model, ops = self.model, self.model.ops
        if self.head_w is None:
            lg = model.logits(self.ws, batch, hid)
            ids = self.ws.next_ids[: lg.shape[0]]
            ops.argmax_rows(lg, ids, model.pdl)
            return ids
        R = batch.logit_rows.numel()
        head_in = hid
        if R != hid.shape[0]:
            head_in = self.ws.head_in[:R]
            torch.index_select(hid, 0, batch.logit_rows.long(), out=head_in)
        lg = self.head_logits[:R]
        model._gemm(head_in, self.head_w, lg)
        ids = self.ws.next_ids[:R]
        ops.argmax_rows(lg, ids, model.pdl)
        ids.copy_(self.head_ids[ids.long()])
        return ids

    def _set_width(self, k: int) -> None:
        """Switches the chained round to k drafts per sequence."""
        if k == self.K:
            return
        if k not in self._width_bufs:
            dev, B = self.device, self.max_batch
            pin = dev.type == "cuda"
            self._width_bufs[k] = (torch.zeros((B, k), dtype=torch.int32, device=dev),
                                   torch.zeros((B, k + 1), dtype=torch.int32, device=dev),
                                   torch.zeros((B, k + 1), dtype=torch.int32, pin_memory=pin),
                                   torch.zeros((B, k), dtype=torch.int32, pin_memory=pin))
        drafts, out_tok, tok_host, draft_host = self._width_bufs[k]
        drafts[:, 0].copy_(self.drafts[:, 0])   # the draft module already proposed the next round's first token
        self.K, self.drafts, self.out_tok, self.tok_host, self.draft_host = k, drafts, out_tok, tok_host, draft_host

    def _mtp_pass(self, batch, hidden_in: torch.Tensor, next_ids: torch.Tensor, seqs: Sequence[int]) -> None:
        """Draft module over `batch`; for the sequences `seqs` (whose last token is a logit row, in order) store
        the first draft token and the module's hidden state."""
        hid = self.model.forward_mtp(self.ws, batch, self.kv_mtp, hidden_in, next_ids)
        if not seqs:
            return
        if self.head_w is not None:
            ids = self._propose(batch, hid)
        else:
            lg = self.model.logits(self.ws, batch, hid)
            ids = self.ws.next_ids[: lg.shape[0]]
            if self._draft_stochastically() and len(self.lengths) > max(seqs):
                self._sample_draft(lg, ids, list(seqs), 0)
            else:
                self.model.ops.argmax_rows(lg, ids, self.model.pdl)
        idx = torch.tensor(list(seqs), dtype=torch.long, device=self.device)
        self.drafts[idx, 0] = ids
        if self.R > 1:
            self.drafts_r[idx, 0] = torch.topk(lg.float(), self.R, dim=-1).indices.to(torch.int32)
        self.mtp_h[idx] = hid.index_select(0, batch.logit_rows.long())

    # ------------------------------------------------------------------ prefill
    def prefill(self, prompts: Sequence[Sequence[int]]) -> List[int]:
        if self.drafter not in ("mtp", "dflash"):
            first = super().prefill(prompts)
            self.history = [list(p) + [t] for p, t in zip(prompts, first)]
            return first
        if len(prompts) > self.max_batch:
            raise ValueError("too many sequences")
        self.reset()
        for r in range(self.max_batch):
            if self.kv_mtp is not None:
                self.kv_mtp.free_row(r)
        if self.dflash is not None:
            self.dflash.reset(range(self.max_batch))
        B = len(prompts)
        for b in range(B):
            self.rows.append(b)
            self.slots.append(self.states.alloc())
            self.lengths.append(0)
            self.kv.ensure(b, len(prompts[b]) + self.K + 2)
            if self.kv_mtp is not None:
                self.kv_mtp.ensure(b, len(prompts[b]) + self.K + 2)
        self.kv.publish()
        if self.kv_mtp is not None:
            self.kv_mtp.publish()
        first = [0] * B
        cursor = [0] * B
        pending = list(range(B))
        while pending:
            budget = self.prefill_chunk
            chunks, owners = [], []
            for b in list(pending):
                if budget == 0 or len(chunks) == self.max_batch:
                    break
                n = min(budget, len(prompts[b]) - cursor[b])
                done = cursor[b] + n == len(prompts[b])
                chunks.append(SeqChunk(self.rows[b], self.slots[b], cursor[b], prompts[b][cursor[b]:cursor[b] + n], done))
                owners.append((b, cursor[b], n, done))
                cursor[b] += n
                budget -= n
                if done:
                    pending.remove(b)
            batch = self.bufs_prefill.build(chunks)
            T = batch.n_tokens
            ids = self.model.forward_greedy(self.ws, batch, self.kv, self.states)
            self.h_keep[:T].copy_(self.ws.normed[:T])
            if ids.numel():
                self.out_host[: ids.numel()].copy_(ids, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            j = 0
            nxt: List[int] = []
            done_seqs = []
            for b, start, n, done in owners:
                if done:
                    first[b] = int(self.out_host[j])
                    j += 1
                    done_seqs.append(b)
                    nxt.extend(list(prompts[b][start + 1:start + n]) + [first[b]])
                else:
                    nxt.extend(prompts[b][start + 1:start + n + 1])
            if self.dflash is not None:
                # the chunk's tokens are committed: their tapped features become draft context
                self.dflash.append_context(self.model.feature_buf[:T], batch.table_row, batch.cache_pos,
                                           {self.rows[b]: start + n for b, start, n, _ in owners})
                continue
            # the draft module reads the same positions: hidden state of p + token p + 1
            self._mtp_pass(batch, self.h_keep[:T], self._upload_next(nxt), done_seqs)
        for b in range(B):
            self.lengths[b] = len(prompts[b])
        self.last_tokens = list(first)
        self.history = [list(p) + [t] for p, t in zip(prompts, first)]
        self.model.status.check("after speculative prefill")
        return first

    # ------------------------------------------------------------------ one round
    def _draft(self, B: int) -> None:
        """Fills self.drafts[:B] (device)."""
        K = self.K
        if self.dflash is not None:
            self.drafts[:B].copy_(self.dflash.propose(self.rows[:B], self.last_tokens[:B], self.lengths[:B]))
            return
        if self.drafter == "mtp":
            for j in range(1, K):
                # position n + j - 1 of the draft module: its own hidden state + the previous draft token
                chunks = [SeqChunk(self.rows[b], self.slots[b], self.lengths[b] + j - 1, [0], True) for b in range(B)]
                batch = self.bufs_draft.build(chunks)
                self.h_in[:B].copy_(self.mtp_h[:B])
                hid = self.model.forward_mtp(self.ws, batch, self.kv_mtp, self.h_in[:B], self.drafts[:B, j - 1].contiguous())
                if self.head_w is not None:
                    ids = self._propose(batch, hid)
                else:
                    lg = self.model.logits(self.ws, batch, hid)
                    ids = self.ws.next_ids[:B]
                    if self._draft_stochastically():
                        self._sample_draft(lg, ids, list(range(B)), j)
                    else:
                        self.model.ops.argmax_rows(lg, ids, self.model.pdl)
                self.drafts[:B, j] = ids
                if self.R > 1:
                    self.drafts_r[:B, j] = torch.topk(lg.float(), self.R, dim=-1).indices.to(torch.int32)
                self.mtp_h[:B].copy_(hid)
            return
        if self.R > 1:
            host = torch.zeros((B, K, self.R), dtype=torch.int32)
            for b in range(B):
                cand = self.tree_hook(b, self.history[b], K, self.R) if self.tree_hook is not None else None
                if cand is None:
                    cand = [[self.last_tokens[b]] * self.R for _ in range(K)]
                host[b] = torch.tensor(cand, dtype=torch.int32)
            self.drafts_r[:B].copy_(host.to(self.device))
            self.drafts[:B].copy_(self.drafts_r[:B, :, 0])
            return
        for b in range(B):
            d = None
            if self.draft_hook is not None:
                d = self.draft_hook(b, self.history[b], K)
            elif self.drafter == "ngram":
                d = ngram_drafter(self.history[b], K)
            elif self.drafter == "lookup":
                d = lookup_drafter(self.history[b], K)   # history chain: K tokens on a full match, a padded probe on a partial one
            if d is None:
                d = [self.last_tokens[b]] * K
            self.draft_host[b] = torch.tensor(list(d)[:K], dtype=torch.int32)
        self.drafts[:B].copy_(self.draft_host[:B], non_blocking=True)

    # ------------------------------------------------------------------ tree round
    def _tree_layout(self):
        """Node order of one verify window: root, then per depth the side branches (ranks 1..R-1) followed by the chain
        node (rank 0), so that every side branch directly follows the state it hangs off."""
        K, R_ = self.K, self.R
        W = 1 + R_ * K
        parent, depth, rank, commit, mask = [-1], [0], [0], [1], [1]
        for d in range(1, K + 1):
            base = 1 + R_ * (d - 1)
            par = R_ * (d - 1)          # chain node of depth d - 1 (0 = root)
            anc = 1
            for dd in range(1, d):
                anc |= 1 << (R_ * dd)
            for j in range(R_):
                r = j + 1 if j < R_ - 1 else 0
                parent.append(par); depth.append(d); rank.append(r); commit.append(1 if r == 0 else 0)
                mask.append(anc | (1 << (base + j)))
        return W, parent, depth, rank, commit, mask

    def decode_round_tree(self) -> List[List[int]]:
        """One round with a draft tree of K depths x R ranks verified in one target pass."""
        B, K, R_ = len(self.rows), self.K, self.R
        ops, dev = self.model.ops, self.device
        W, parent, depth, rank, commit, mask = self._tree_layout()
        for b, r in enumerate(self.rows):
            self.kv.ensure(r, self.lengths[b] + W + 1)
            if self.kv_mtp is not None:
                self.kv_mtp.ensure(r, self.lengths[b] + K + 2)
        self.kv.publish()
        if self.kv_mtp is not None:
            self.kv_mtp.publish()
        self._draft(B)
        chunks = [SeqChunk(self.rows[b], self.slots[b], self.lengths[b], [self.last_tokens[b]] + [0] * (W - 1), True, True)
                  for b in range(B)]
        batch = self.bufs_verify.build(chunks)
        T = B * W
        # node tokens: drafts_r[b, depth - 1, rank]
        d_idx = torch.tensor(depth[1:], device=dev) - 1
        r_idx = torch.tensor(rank[1:], device=dev)
        batch.ids.view(B, W)[:, 1:] = self.drafts_r[:B][:, d_idx, r_idx]
        n0 = torch.tensor(self.lengths[:B], dtype=torch.int32, device=dev)[:, None]
        batch.rope_pos.view(B, W).copy_(n0 + torch.tensor(depth, dtype=torch.int32, device=dev)[None])
        batch.kv_len.view(B, W).copy_((n0 + W).expand(B, W))
        offs = (torch.arange(B, dtype=torch.int32, device=dev) * W)[:, None]
        par = torch.tensor(parent, dtype=torch.int32, device=dev)[None].expand(B, W)
        batch.tree_parent = torch.where(par >= 0, par + offs, par).reshape(-1).contiguous()
        batch.tree_commit = torch.tensor(commit, dtype=torch.uint8, device=dev).repeat(B)
        batch.tree_mask = torch.tensor(mask, dtype=torch.int64, device=dev).repeat(B)
        batch.tree_base = n0.expand(B, W).reshape(-1).contiguous()
        hidden = self.model.forward_hidden(self.ws, batch, self.kv, self.states, write_state=False, rec=self.rec)
        self.h_keep[:T].copy_(hidden)
        lg = self.model.logits(self.ws, batch, hidden)
        target = self.ws.next_ids[:T]
        ops.argmax_rows(lg, target, self.model.pdl)
        n_acc = torch.empty(B, dtype=torch.int32, device=dev)
        out_tok = torch.empty((B, K + 1), dtype=torch.int32, device=dev)
        out_node = torch.empty((B, K + 1), dtype=torch.int32, device=dev)
        ops.accept_greedy_tree(target.view(B, W), batch.ids.view(B, W), par.contiguous(), K, n_acc, out_tok, out_node)
        acc_h, tok_h, node_h = n_acc.cpu(), out_tok.cpu(), out_node.cpu()   # (synchronises)
        emitted: List[List[int]] = []
        accepted = torch.zeros((B, W), dtype=torch.uint8)
        last = torch.zeros(B, dtype=torch.int32)
        src = torch.full((B, K), -1, dtype=torch.int32)
        dst = torch.full((B, K), -1, dtype=torch.int32)
        path_rows: List[int] = []
        for b in range(B):
            m = int(acc_h[b])
            emitted.append([int(v) for v in tok_h[b, : m + 1]])
            accepted[b, 0] = 1
            last[b] = b * W
            path_rows.append(b * W)
            for d in range(m):
                node = int(node_h[b, d])
                accepted[b, node] = 1
                last[b] = b * W + node
                path_rows.append(b * W + node)
                src[b, d] = self.lengths[b] + node
                dst[b, d] = self.lengths[b] + d + 1
            self.accepted += m
            self.emitted += m + 1
        self.rounds += 1
        # state: replay with the accepted path as the only committing tokens; KV: accepted rows to their final places
        self.model.fold_gdn_tree(self.ws, batch, self.states, self.rec, accepted.view(-1).to(dev), last.to(dev))
        src_d, dst_d = src.to(dev), dst.to(dev)
        trow = torch.tensor(self.rows[:B], dtype=torch.int32, device=dev)
        g = self.model.g
        for planes in self.kv.layers:
            ops.kv_move_rows(self.kv.table, trow, src_d, dst_d, planes.k_codes, planes.v_codes, planes.k_scales,
                             planes.v_scales, self.kv.page_size, g.n_kv_heads, self.cfg.head_dim, planes.fmt, planes.group)
        if self.drafter == "mtp":
            chunks, nxt = [], []
            for b in range(B):
                chunks.append(SeqChunk(self.rows[b], self.slots[b], self.lengths[b], [0] * len(emitted[b]), True))
                nxt.extend(emitted[b])
            cb = self.bufs_catch.build(chunks)
            idx = torch.tensor(path_rows, dtype=torch.long, device=dev)
            Tc = len(path_rows)
            torch.index_select(self.h_keep[:T], 0, idx, out=self.h_in[:Tc])
            self._mtp_pass(cb, self.h_in[:Tc], self._upload_next(nxt), list(range(B)))
        for b in range(B):
            self.lengths[b] += len(emitted[b])
            self.last_tokens[b] = emitted[b][-1]
            self.history[b].extend(emitted[b])
        return emitted

    # ------------------------------------------------------------------ chained round as one graph
    def _graph_round_ok(self) -> bool:
        """A chained round can be replayed as a graph when nothing in it needs the host: greedy verification and a
        drafter that either runs on the device (the draft module) or proposes before the round (hook, n-gram)."""
        if not self.use_graph or self.R > 1 or self.dflash is not None:
            return False
        sps = self.sampling if isinstance(self.sampling, (list, tuple)) else [self.sampling]
        return all(sp is None or sp.greedy for sp in sps)

    def _round_descriptors(self, B: int):
        K = self.K
        bd = self.bufs_draft.build([SeqChunk(self.rows[b], self.slots[b], self.lengths[b], [0], True) for b in range(B)])
        bv = self.bufs_verify.build([SeqChunk(self.rows[b], self.slots[b], self.lengths[b],
                                              [self.last_tokens[b]] + [0] * K, True, True) for b in range(B)])
        return bd, bv

    def _round_body(self, B: int, bd, bv) -> None:
        """The device work of one chained greedy round, free of host reads.  The draft module's catch-up runs over
        all K + 1 verify rows of every sequence: rows past the accepted prefix compute values nobody reads (their
        cache positions are rewritten by the next round before any query can see them), and the row that carries the
        next first draft is picked on the device from the accepted length."""
        K, ops, model, ws = self.K, self.model.ops, self.model, self.ws
        T = B * (K + 1)
        if self.drafter == "mtp":
            for j in range(1, K):
                self.h_in[:B].copy_(self.mtp_h[:B])
                self.draft_col[:B].copy_(self.drafts[:B, j - 1])
                hid = model.forward_mtp(ws, bd, self.kv_mtp, self.h_in[:B], self.draft_col[:B])
                self.drafts[:B, j] = self._propose(bd, hid)
                self.mtp_h[:B].copy_(hid)
                bd.cache_pos.add_(1)
                bd.kv_len.add_(1)
                bd.rope_pos.add_(1)
        bv.ids.view(B, K + 1)[:, 1:] = self.drafts[:B]
        hidden = model.forward_hidden(ws, bv, self.kv, self.states, write_state=False, rec=self.rec)
        self.h_keep[:T].copy_(hidden)
        lg = model.logits(ws, bv, hidden)
        target = ws.next_ids[:T]
        ops.argmax_rows(lg, target, model.pdl)
        ops.accept_greedy_chain(target.view(B, K + 1), self.drafts[:B], self.n_acc[:B], self.out_tok[:B])
        torch.add(bv.cu_seqlens[:B], self.n_acc[:B], out=self.catch_rows[:B])
        torch.add(self.catch_rows[:B], 1, out=self.seq_end[:B])
        model.fold_gdn(ws, bv, self.states, self.rec, self.seq_end[:B])
        if self.drafter == "mtp":
            cb = replace(bv, logit_rows=self.catch_rows[:B])
            torch.clamp(self.out_tok[:B].view(-1), min=0, out=self.next_dev[:T])
            self.h_in[:T].copy_(self.h_keep[:T])
            hid = model.forward_mtp(ws, cb, self.kv_mtp, self.h_in[:T], self.next_dev[:T])
            torch.index_select(hid, 0, self.catch_rows[:B].long(), out=self.mtp_h[:B])
            self.drafts[:B, 0] = self._propose(cb, hid)

    def _round_graph(self, B: int, bucket: int):
        key = (B, bucket, self.K)
        if key in self._round_graphs:
            return self._round_graphs[key]
        bd, bv = self._round_descriptors(B)
        bd.max_kv_len = bv.max_kv_len = bucket   # bake the bucket's split geometry, not this round's
        keep = (self.mtp_h.clone(), self.drafts.clone())

        def restore():
            self._rollback_states()
            self.mtp_h.copy_(keep[0])
            self.drafts.copy_(keep[1])
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):   # warm-up outside capture; a round moves the recurrent state and the draft inputs
                self._snapshot_states()
                self.bufs_draft.dev.copy_(self.bufs_draft.host, non_blocking=True)
                self._round_body(B, bd, bv)
                restore()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(self.device)
        self.bufs_draft.dev.copy_(self.bufs_draft.host, non_blocking=True)
        graph = torch.cuda.CUDAGraph()
        self._snapshot_states()
        with torch.cuda.graph(graph):
            self._round_body(B, bd, bv)
        restore()
        self._round_graphs[key] = (graph, bd, bv)
        self._fresh_graph = True
        return self._round_graphs[key]

    def _decode_round_graph(self) -> List[List[int]]:
        B, K = len(self.rows), self.K
        for b, r in enumerate(self.rows):
            self.kv.ensure(r, self.lengths[b] + K + 2)
            if self.kv_mtp is not None:
                self.kv_mtp.ensure(r, self.lengths[b] + K + 2)
        self.kv.publish()
        if self.kv_mtp is not None:
            self.kv_mtp.publish()
        if self.drafter != "mtp":
            self._draft(B)   # host proposals: one upload before the graph
        graph, _, _ = self._round_graph(B, context_bucket(max(self.lengths) + K + 2))
        self._round_descriptors(B)
        graph.replay()
        self.acc_host[:B].copy_(self.n_acc[:B], non_blocking=True)
        self.tok_host[:B].copy_(self.out_tok[:B], non_blocking=True)
        t_wait = time.perf_counter()
        torch.cuda.current_stream().synchronize()
        self.device_wait_s += time.perf_counter() - t_wait
        emitted: List[List[int]] = []
        for b in range(B):
            m = int(self.acc_host[b])
            toks = [int(v) for v in self.tok_host[b, : m + 1]]
            emitted.append(toks)
            self.accepted += m
            self.emitted += m + 1
            self.lengths[b] += m + 1
            self.last_tokens[b] = toks[-1]
            self.history[b].extend(toks)
        self.rounds += 1
        return emitted

    def _accept_log(self, emitted: List[List[int]]) -> List[List[int]]:
        """`NINFER_ACCEPTLOG=<path>`: one JSON line per round (round, drafts per sequence, tree ranks, accepted drafts
        of every sequence), for acceptance studies without touching the request log."""
        path = os.environ.get("NINFER_ACCEPTLOG", "")
        if path:
            import json
            with open(path, "a", encoding="utf-8") as f:
                f.write(json.dumps({"round": self.rounds, "width": self.K, "ranks": self.R, "drafter": self.drafter,
                                    "accepted": [len(e) - 1 for e in emitted]}) + "\n")
        return emitted

    def decode_round(self) -> List[List[int]]:
        """One draft-verify round; returns the tokens emitted for every sequence (1..K+1 each)."""
        if self.R > 1:
            return self._accept_log(self.decode_round_tree())
        ctl = self.width_ctl
        if ctl is None:
            return self._accept_log(self._decode_round_graph() if self._graph_round_ok() else self._decode_round_eager())
        self._set_width(ctl.width)
        self._fresh_graph = False
        t0 = time.perf_counter()
        emitted = self._decode_round_graph() if self._graph_round_ok() else self._decode_round_eager()
        # the round ends with a stream synchronisation, so the host clock brackets the whole round; a round that
        # captured its graph first says nothing about the cost of its width
        ms = None if self._fresh_graph else (time.perf_counter() - t0) * 1e3
        ctl.observe_round([len(e) - 1 for e in emitted], self.K, ms)
        return self._accept_log(emitted)

    def _decode_round_eager(self) -> List[List[int]]:
        B, K = len(self.rows), self.K
        ops = self.model.ops
        for b, r in enumerate(self.rows):
            self.kv.ensure(r, self.lengths[b] + K + 2)
            if self.kv_mtp is not None:
                self.kv_mtp.ensure(r, self.lengths[b] + K + 2)
        self.kv.publish()
        if self.kv_mtp is not None:
            self.kv_mtp.publish()
        self._draft(B)
        # ---- verify: [t, d_1..d_K] per sequence in one ragged target pass ----
        chunks = [SeqChunk(self.rows[b], self.slots[b], self.lengths[b], [self.last_tokens[b]] + [0] * K, True, True)
                  for b in range(B)]
        batch = self.bufs_verify.build(chunks)
        T = B * (K + 1)
        batch.ids.view(B, K + 1)[:, 1:] = self.drafts[:B]
        hidden = self.model.forward_hidden(self.ws, batch, self.kv, self.states, write_state=False, rec=self.rec)
        self.h_keep[:T].copy_(hidden)
        lg = self.model.logits(self.ws, batch, hidden)
        target = self.ws.next_ids[:T]
        sps = self.sampling if isinstance(self.sampling, (list, tuple)) else [self.sampling] * B
        if all(sp is None or sp.greedy for sp in sps):
            ops.argmax_rows(lg, target, self.model.pdl)
        else:
            # speculative sampling: column j draws against draft j + 1 (the last column has no draft: bonus token);
            # a rejected column already holds its replacement, so the chain rule below applies unchanged.  Rows of a
            # greedy sequence carry temperature 0 and fall back to arg-max acceptance inside the same kernel.
            dev = self.device
            d = torch.full((B, K + 1), -1, dtype=torch.int32, device=dev)
            d[:, :K] = self.drafts[:B]
            pos = torch.tensor([self.lengths[b] + j + 1 for b in range(B) for j in range(K + 1)], dtype=torch.int32, device=dev)

            def rows(get, dtype):
                return torch.tensor([get(sps[b]) for b in range(B) for _ in range(K + 1)], dtype=dtype, device=dev)
            ops.sample_rows(lg, rows(lambda sp: 0.0 if sp is None else sp.temperature, torch.float32),
                            rows(lambda sp: 1 if sp is None else sp.top_k, torch.int32),
                            rows(lambda sp: 1.0 if sp is None else sp.top_p, torch.float32),
                            rows(lambda sp: 0.0 if sp is None else sp.min_p, torch.float32), None, None, None,
                            rows(lambda sp: 0 if sp is None else sp.seed, torch.int64), pos, 0, target, None,
                            d.view(-1), torch.empty(T, dtype=torch.int32, device=dev),
                            *((self.q_ids[:B].reshape(T, -1), self.q_probs[:B].reshape(T, -1))
                              if self._draft_stochastically() else ()))
        # ---- accept + fold ----
        ops.accept_greedy_chain(target.view(B, K + 1), self.drafts[:B], self.n_acc[:B], self.out_tok[:B])
        seq_end = (batch.cu_seqlens[:B] + self.n_acc[:B] + 1).to(torch.int32)
        self.model.fold_gdn(self.ws, batch, self.states, self.rec, seq_end)
        self.acc_host[:B].copy_(self.n_acc[:B], non_blocking=True)
        self.tok_host[:B].copy_(self.out_tok[:B], non_blocking=True)
        t_wait = time.perf_counter()
        torch.cuda.current_stream().synchronize()
        self.device_wait_s += time.perf_counter() - t_wait
        emitted: List[List[int]] = []
        for b in range(B):
            m = int(self.acc_host[b])
            toks = [int(v) for v in self.tok_host[b, : m + 1]]
            emitted.append(toks)
            self.accepted += m
            self.emitted += m + 1
        self.rounds += 1
        # ---- draft-module catch-up over the accepted positions with the target's hidden states ----
        if self.drafter == "mtp":
            chunks, rows, nxt = [], [], []
            for b in range(B):
                m1 = len(emitted[b])
                chunks.append(SeqChunk(self.rows[b], self.slots[b], self.lengths[b], [0] * m1, True))
                rows.extend(range(b * (K + 1), b * (K + 1) + m1))
                nxt.extend(emitted[b])
            cb = self.bufs_catch.build(chunks)
            idx = torch.tensor(rows, dtype=torch.long, device=self.device)
            Tc = len(rows)
            torch.index_select(self.h_keep[:T], 0, idx, out=self.h_in[:Tc])
            self._mtp_pass(cb, self.h_in[:Tc], self._upload_next(nxt), list(range(B)))
        if self.dflash is not None:
            # the features of the positions that were just committed (verify rows 0..m of every sequence) extend the
            # draft context; they sit at cache positions lengths[b] + j
            rows, trow, pos, ends = [], [], [], {}
            for b in range(B):
                m1 = len(emitted[b])
                rows.extend(range(b * (K + 1), b * (K + 1) + m1))
                trow.extend([self.rows[b]] * m1)
                pos.extend(range(self.lengths[b], self.lengths[b] + m1))
                ends[self.rows[b]] = self.lengths[b] + m1
            idx = torch.tensor(rows, dtype=torch.long, device=self.device)
            feats = self.model.feature_buf[:T].index_select(0, idx)
            self.dflash.append_context(feats, torch.tensor(trow, dtype=torch.int32, device=self.device),
                                       torch.tensor(pos, dtype=torch.int32, device=self.device), ends)
        for b in range(B):
            self.lengths[b] += len(emitted[b])
            self.last_tokens[b] = emitted[b][-1]
            self.history[b].extend(emitted[b])
        return emitted

    def generate(self, prompts: Sequence[Sequence[int]], n_new: int) -> List[List[int]]:
        first = self.prefill(prompts)
        out = [[t] for t in first]
        while min(len(o) for o in out) < n_new:
            for b, toks in enumerate(self.decode_round()):
                out[b].extend(toks)
        self.model.status.check("after speculative decode")
        return [o[:n_new] for o in out]

    @property
    def tokens_per_round(self) -> float:
        B = max(1, len(self.rows))
        return self.emitted / max(1, self.rounds * B)


class SpeculativeProgram:
    """Lane-based Program (the Engine's interface) on top of the speculative generator: MTP chain drafts, one verify
    pass per round, several committed tokens per lane and round.  Lanes join and leave between rounds; the
    generator's per-sequence arrays are rebuilt from the lanes before every round, and the two pieces of draft state
    that persist between rounds (first draft token, draft-module hidden state) are kept per block-table row.

    Reference: ProgramImpl's speculative decode rounds (src/targets/qwen3_6/impl/runtime/mtp_impl.h,
    speculative_target_impl.h) behind the same Program API as ordinary decode."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], device, max_lanes: int = 8,
                 max_context: int = 4096, draft_tokens: int = 3, **kw):
        from .program import Lane, ProgramBase, SamplingParams  # noqa: F401
        self.gen = SpeculativeGenerator(cfg, weights, device, max_lanes, max_context, draft_tokens=draft_tokens,
                                        drafter="mtp", **kw)
        self.cfg, self.max_lanes, self.max_context = cfg, max_lanes, max_context
        self.K = draft_tokens
        self._base = ProgramBase(cfg, max_lanes, max_context)
        self.lanes = self._base.lanes
        self.checkpoints: list = []
        h = cfg.hidden
        self.row_draft = torch.zeros(max_lanes, dtype=torch.int32, device=self.gen.device)
        self.row_mtp_h = torch.zeros((max_lanes, h), dtype=torch.bfloat16, device=self.gen.device)
        # the first draft token's distribution q (stochastic drafts) belongs to the row as well
        self.row_q_ids = torch.full((max_lanes, self.gen.q_ids.shape[2]), -1, dtype=torch.int32, device=self.gen.device)
        self.row_q_probs = torch.zeros((max_lanes, self.gen.q_ids.shape[2]), dtype=torch.float32, device=self.gen.device)

    @property
    def device_wait_s(self) -> float:
        return self.gen.device_wait_s

    speculative_backend = "mtp"

    def force_next_token(self, lane, token: int) -> None:
        """The next round verifies from `token`; the draft module's first proposal was made for the sampled token and
        is simply rejected if it no longer fits."""
        lane.last_token = int(token)

    @property
    def draft_window(self) -> int:
        """Drafts per sequence in the round that just ran (the width in force: it moves under the adaptive controller)."""
        return self.gen.K

    # ---- Program API ----
    def free_lanes(self) -> int:
        return len(self._base._free_rows)

    def can_admit(self, n_prompt: int, max_new: int) -> bool:
        g = self.gen
        need = (n_prompt + max_new + self.K + 2 + g.page_size - 1) // g.page_size
        return bool(self._base._free_rows) and n_prompt + max_new + self.K + 2 <= self.max_context and \
            g.kv.pool.free_pages >= need and g.kv_mtp.pool.free_pages >= need

    def open(self, prompt, sampling=None, session=None):
        from .engine import RequestError
        from .program import Lane, SamplingParams
        sampling = sampling or SamplingParams()
        if getattr(sampling, "presence_penalty", 0.0) or getattr(sampling, "frequency_penalty", 0.0):
            # verification samples without per-lane token counts, so a penalty would silently change the
            # distribution between the speculative and the ordinary program: refuse instead
            raise RequestError("presence / frequency penalties are not supported by the speculative program")
        if not self._base._free_rows:
            raise MemoryError("no free lane")
        slot = self.gen.states.alloc()      # before the row is taken: a failure here must not leak the row
        row = self._base._free_rows.pop()
        lane = Lane(self._base._next_id, row, slot, list(prompt), 0, sampling)
        self._base._next_id += 1
        self.lanes[lane.lane_id] = lane
        return lane

    def close(self, lane) -> None:
        if self.lanes.pop(lane.lane_id, None) is None:
            return
        self.gen.kv.free_row(lane.row)
        self.gen.kv_mtp.free_row(lane.row)
        self.gen.states.release(lane.slot)
        self._base._free_rows.append(lane.row)

    def checkpoint(self, lane, session, kind) -> bool:
        return False   # the draft module's cache is not part of a frontier yet: no prefix reuse in speculative mode

    def prefill_step(self, lane, budget: int):
        g = self.gen
        n = min(budget, g.prefill_chunk, len(lane.tokens) - lane.n_cached)
        done = lane.n_cached + n == len(lane.tokens)
        for cache in (g.kv, g.kv_mtp):
            cache.ensure(lane.row, lane.n_cached + n + self.K + 2)
            cache.publish()
        chunk = SeqChunk(lane.row, lane.slot, lane.n_cached, lane.tokens[lane.n_cached:lane.n_cached + n], done)
        batch = g.bufs_prefill.build([chunk])
        ids = g.model.forward_greedy(g.ws, batch, g.kv, g.states)
        g.h_keep[:n].copy_(g.ws.normed[:n])
        first = None
        nxt = list(lane.tokens[lane.n_cached + 1:lane.n_cached + n + 1])
        if done:
            g.out_host[:1].copy_(ids[:1], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            first = int(g.out_host[0])
            nxt = nxt + [first]
        # the draft module reads the same positions (hidden state of p + token p + 1); the first draft of a finished
        # prompt is drawn under this lane's own sampling parameters
        if done:
            g.sampling, g.lengths = [lane.sampling], [lane.n_cached + n]
        g._mtp_pass(batch, g.h_keep[:n], g._upload_next(nxt), [0] if done else [])
        if done:
            self.row_draft[lane.row] = g.drafts[0, 0]
            self.row_mtp_h[lane.row].copy_(g.mtp_h[0])
            self.row_q_ids[lane.row].copy_(g.q_ids[0, 0])
            self.row_q_probs[lane.row].copy_(g.q_probs[0, 0])
        lane.n_cached += n
        g.model.status.check("after speculative prefill")
        if done:
            lane.last_token = first
        return first

    def decode_round(self, lanes):
        g = self.gen
        B = len(lanes)
        if B == 0:
            return []
        rows = torch.tensor([l.row for l in lanes], dtype=torch.long, device=g.device)
        g.rows = [l.row for l in lanes]
        g.slots = [l.slot for l in lanes]
        g.lengths = [l.n_cached for l in lanes]
        g.last_tokens = [l.last_token for l in lanes]
        g.history = [list(l.tokens) + [l.last_token] for l in lanes]
        g.sampling = [l.sampling for l in lanes]
        g.drafts[:B, 0] = self.row_draft[rows]
        g.mtp_h[:B] = self.row_mtp_h[rows]
        g.q_ids[:B, 0] = self.row_q_ids[rows]
        g.q_probs[:B, 0] = self.row_q_probs[rows]
        emitted = g.decode_round()
        self.row_draft[rows] = g.drafts[:B, 0]
        self.row_mtp_h[rows] = g.mtp_h[:B]
        self.row_q_ids[rows] = g.q_ids[:B, 0]
        self.row_q_probs[rows] = g.q_probs[:B, 0]
        for l, toks in zip(lanes, emitted):
            l.tokens.append(l.last_token)
            l.tokens.extend(toks[:-1])
            l.n_cached += len(toks)
            l.last_token = toks[-1]
        return emitted
