"""Step descriptors: pinned host staging + one H2D copy per step.

All per-token / per-sequence int32 arrays of a step live in ONE packed buffer
(host pinned + device twin) with fixed offsets, so that (a) a step uploads its
inputs with a single async copy, and (b) the device views have stable addresses
and can be baked into a CUDA graph.  This is the counterpart of the reference's
pinned "ingress" struct (src/targets/qwen3_6/impl/runtime/program_impl.h:18436-18452).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch

from ..models.hybrid import StepBatch


@dataclass
class SeqChunk:
    """Tokens of one sequence processed in this step."""
    table_row: int       # KV block-table row
    state_slot: int      # GDN state slot
    start_pos: int       # cache position of the first token
    tokens: Sequence[int]
    want_logits: bool = True   # logits for the chunk's last token
    all_logits: bool = False   # logits for every token of the chunk (speculative verify)
    positions: object = None   # optional int [n, 3] rope positions (multimodal prefill); default = cache positions


class StepBuffers:
    def __init__(self, max_tokens: int, max_seqs: int, device, mrope: bool = False, attn_block_tokens: int = 16,
                 max_logit_rows: int = 0):
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        n_logit_rows = max(max_seqs, max_logit_rows)
        self.device = torch.device(device)
        self.pos_axes = 3 if mrope else 1
        T, B = max_tokens, max_seqs
        self.attn_block_tokens = max(1, attn_block_tokens)
        NB = (T + self.attn_block_tokens - 1) // self.attn_block_tokens + B
        sizes = [("ids", T), ("token_seq", T), ("table_row", T), ("cache_pos", T), ("rope_pos", T * self.pos_axes),
                 ("kv_len", T), ("cu_seqlens", B + 1), ("state_slot", B), ("logit_rows", n_logit_rows), ("qblk_start", NB), ("qblk_count", NB)]
        self.offsets = {}
        off = 0
        for name, n in sizes:
            self.offsets[name] = (off, n)
            off += (n + 3) // 4 * 4  # keep every view 16-byte aligned
        self.total = off
        pin = self.device.type == "cuda"
        self.host = torch.zeros(off, dtype=torch.int32, pin_memory=pin)
        self.dev = torch.zeros(off, dtype=torch.int32, device=self.device)
        self._np = self.host.numpy()

    def _hview(self, name: str, n: int):
        off, cap = self.offsets[name]
        assert n <= cap, f"{name}: {n} > capacity {cap}"
        return self._np[off:off + n]

    def _dview(self, name: str, n: int) -> torch.Tensor:
        off, _ = self.offsets[name]
        return self.dev[off:off + n]

    def h2d_bytes(self) -> int:
        return self.total * 4

    def build(self, chunks: List[SeqChunk], upload: bool = True, rope_delta: Sequence[int] | None = None) -> StepBatch:
        T = sum(len(c.tokens) for c in chunks)
        B = len(chunks)
        if T > self.max_tokens or B > self.max_seqs:
            raise ValueError(f"step ({T} tokens, {B} seqs) exceeds buffers ({self.max_tokens}, {self.max_seqs})")
        ids, tseq, trow = self._hview("ids", T), self._hview("token_seq", T), self._hview("table_row", T)
        cpos, kvl = self._hview("cache_pos", T), self._hview("kv_len", T)
        rpos = self._hview("rope_pos", T * self.pos_axes)
        cu, slot = self._hview("cu_seqlens", B + 1), self._hview("state_slot", B)
        lrows = self._hview("logit_rows", sum(len(c.tokens) if c.all_logits else 1 for c in chunks))
        t = 0
        n_logit = 0
        qt = self.attn_block_tokens
        blk_s, blk_c = [], []
        max_kv = 1
        cu[0] = 0
        for b, c in enumerate(chunks):
            n = len(c.tokens)
            ids[t:t + n] = c.tokens
            tseq[t:t + n] = b
            trow[t:t + n] = c.table_row
            pos = range(c.start_pos, c.start_pos + n)
            cpos[t:t + n] = pos
            kvl[t:t + n] = range(c.start_pos + 1, c.start_pos + n + 1)
            d = rope_delta[b] if rope_delta is not None and b < len(rope_delta) else 0
            if c.positions is not None:
                if self.pos_axes != 3:
                    raise ValueError("explicit positions need three-axis step buffers")
                rpos[3 * t:3 * (t + n)] = np.asarray(c.positions, dtype=np.int32).reshape(-1)
            elif self.pos_axes == 1:
                rpos[t:t + n] = range(c.start_pos + d, c.start_pos + d + n)
            else:
                for a in range(3):
                    rpos[3 * t + a:3 * (t + n):3] = range(c.start_pos + d, c.start_pos + d + n)
            slot[b] = c.state_slot
            for o in range(0, n, qt):
                blk_s.append(t + o)
                blk_c.append(min(qt, n - o))
            t += n
            cu[b + 1] = t
            if c.all_logits:
                lrows[n_logit:n_logit + n] = range(t - n, t)
                n_logit += n
            elif c.want_logits:
                lrows[n_logit] = t - 1
                n_logit += 1
            max_kv = max(max_kv, c.start_pos + n)
        nb = len(blk_s)
        self._hview("qblk_start", nb)[:] = blk_s
        self._hview("qblk_count", nb)[:] = blk_c
        if upload:
            self.dev.copy_(self.host, non_blocking=True)
        rp = self._dview("rope_pos", T * self.pos_axes)
        if self.pos_axes == 3:
            rp = rp.view(T, 3)
        return StepBatch(ids=self._dview("ids", T), token_seq=self._dview("token_seq", T),
                         table_row=self._dview("table_row", T), cache_pos=self._dview("cache_pos", T), rope_pos=rp,
                         kv_len=self._dview("kv_len", T), cu_seqlens=self._dview("cu_seqlens", B + 1),
                         state_slot=self._dview("state_slot", B), logit_rows=self._dview("logit_rows", n_logit),
                         max_kv_len=max_kv, n_tokens=T, n_seqs=B,
                         one_token_per_seq=all(len(c.tokens) == 1 for c in chunks),
                         qblk_start=self._dview("qblk_start", nb), qblk_count=self._dview("qblk_count", nb))
