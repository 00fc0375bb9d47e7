"""Block selector for selected-block attention: which 4-token blocks of its history a decode query attends to.

Every complete block of four consecutive keys is summarised by the mean of its (dequantised) K rows per KV head; a
query scores a block by the largest dot product of its GQA group's heads with that summary, keeps the `budget` best
blocks and always keeps the most recent `recent` blocks (the local window) and the first `sink` blocks.  The result
is the `(sel_blocks, sel_count)` pair that ``torch.ops.nfb200.paged_attention`` takes; the incomplete last block is
added by the kernel itself.  Plain tensor code: the selector runs once per layer and round on summaries that are a
quarter of the keys, the attention over the selection is the hand-written kernel.

Reference: the query-selected sparse attention of the FlashNext target (src/targets/qwen3_8_flash_next, selection
feeding include/ninfer/ops/selected_block_attention.h).
"""
from __future__ import annotations

from typing import Tuple

import torch

BLOCK = 4


def block_summaries(k: torch.Tensor) -> torch.Tensor:
    """k: [n_keys, n_kv_heads, D] -> [n_keys // 4, n_kv_heads, D], the mean key of every complete block."""
    n = (k.shape[0] // BLOCK) * BLOCK
    return k[:n].to(torch.float32).reshape(n // BLOCK, BLOCK, k.shape[1], k.shape[2]).mean(1)


def select_blocks(q: torch.Tensor, summaries: torch.Tensor, kv_len: int, budget: int, recent: int = 4, sink: int = 1,
                  max_blocks: int = 512) -> Tuple[torch.Tensor, int]:
    """q: [n_q_heads, D] of one query token; summaries: [n_blocks_total, n_kv_heads, D]; kv_len: visible keys.
    Returns (block ids int32 [max_blocks], count): ids ascending, every id below kv_len // 4."""
    complete = min(kv_len // BLOCK, summaries.shape[0])
    if complete <= 0:
        return torch.zeros(max_blocks, dtype=torch.int32, device=q.device), 0
    Hq, D = q.shape
    Hkv = summaries.shape[1]
    g = Hq // Hkv
    s = summaries[:complete].to(torch.float32)                                   # [blocks, Hkv, D]
    scores = torch.einsum("hgd,bhd->bhg", q.to(torch.float32).reshape(Hkv, g, D), s).amax(dim=(1, 2))   # [blocks]
    keep = torch.zeros(complete, dtype=torch.bool, device=q.device)
    keep[: min(sink, complete)] = True
    keep[max(0, complete - recent):] = True
    want = min(max_blocks, max(budget, int(keep.sum())))
    extra = want - int(keep.sum())
    if extra > 0:
        masked = scores.masked_fill(keep, float("-inf"))
        top = torch.topk(masked, min(extra, complete - int(keep.sum()))).indices if complete > int(keep.sum()) else None
        if top is not None:
            keep[top] = True
    ids = torch.nonzero(keep).flatten().to(torch.int32)
    out = torch.zeros(max_blocks, dtype=torch.int32, device=q.device)
    out[: ids.numel()] = ids
    return out, int(ids.numel())
