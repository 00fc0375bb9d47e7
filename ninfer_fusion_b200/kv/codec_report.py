"""CPU KV-codec comparison on a paged GQA decode workload.

Workload: 1 layer, 8 query heads / 2 KV heads, head_dim 128, 4 sequences of
length 37 / 256 / 1000 / 2048, page size 16; Q/K/V bf16 drawn N(0,1) from a
seed with 4 random K channels scaled x8 as outliers.  KV is stored as bf16,
fp8-E4M3 with a per-row scale and int8 with group-32 scales (nvfp4, nvfp4 with the K
row scale and the E8-lattice K tier are reported too); the report gives the attention-output max / mean absolute error of each
codec against bf16 storage and the bytes per token.

Run: ``python -m ninfer_fusion_b200.kv.codec_report``
"""
from __future__ import annotations

import json
import math
from typing import Dict, List

import torch

from ..ops import reference as R


def paged_decode_reference(q: torch.Tensor, k_rows: torch.Tensor, v_rows: torch.Tensor, table: List[int],
                           page_size: int, kv_len: int) -> torch.Tensor:
    """q [Hq, D]; k_rows/v_rows [n_pages, Hkv, P, D] dequantised page planes; table = page ids of the sequence."""
    n = (kv_len + page_size - 1) // page_size
    k = torch.cat([k_rows[table[i]].permute(1, 0, 2) for i in range(n)], 0)[:kv_len]  # [L, Hkv, D]
    v = torch.cat([v_rows[table[i]].permute(1, 0, 2) for i in range(n)], 0)[:kv_len]
    return R.gqa_attention(q[None], k, v, torch.tensor([kv_len]), 1.0 / math.sqrt(q.shape[-1]))[0]


def run(seed: int = 0, n_q_heads: int = 8, n_kv_heads: int = 2, head_dim: int = 128,
        lengths=(37, 256, 1000, 2048), page_size: int = 16, int8_group: int = 32) -> Dict:
    g = torch.Generator().manual_seed(seed)
    D = head_dim
    outliers = torch.randperm(D, generator=g)[:4]
    # "+hadamard": K (and the query) rotated by the normalised Hadamard matrix before K is quantised, which spreads
    # the outlier channels over the row (the reference's fixed orthogonal K frame, src/ops/kv_cache/hadamard_d256.cuh)
    formats = [("bf16", R.KV_BF16, D), ("fp8-e4m3-row", R.KV_FP8_ROW, D), ("fp8-e4m3-row+hadamard", R.KV_FP8_ROW, D),
               (f"int8-g{int8_group}", R.KV_INT8_GROUP, int8_group), ("nvfp4-g16", R.KV_NVFP4, 16),
               # nvfp4 with the K row scale (per-channel multipliers solved from the sequence's own keys, K x s stored,
               # q / s applied: kv/rowscale.py) and the E8-lattice K tier beside an nvfp4 V (kv/e8_lattice.py)
               ("nvfp4-g16+rowscale", R.KV_NVFP4, 16), ("e8-rk4v4", R.KV_NVFP4, 16),
               ("e8-rk4v4+hadamard", R.KV_NVFP4, 16)]
    Hn = R.hadamard_matrix(D)
    seqs = []
    n_pages_total = sum((n + page_size - 1) // page_size for n in lengths)
    perm = torch.randperm(n_pages_total, generator=g).tolist()
    cursor = 0
    for n in lengths:
        k = torch.randn(n, n_kv_heads, D, generator=g)
        k[:, :, outliers] *= 8.0
        v = torch.randn(n, n_kv_heads, D, generator=g)
        q = torch.randn(n_q_heads, D, generator=g)
        np_ = (n + page_size - 1) // page_size
        seqs.append((R.bf16_round(q), R.bf16_round(k), R.bf16_round(v), perm[cursor:cursor + np_]))
        cursor += np_
    report = {"workload": {"q_heads": n_q_heads, "kv_heads": n_kv_heads, "head_dim": D, "lengths": list(lengths),
                           "page_size": page_size, "outlier_channels": outliers.tolist()}, "codecs": {}}
    outs = {}
    for name, fmt, group in formats:
        k_pages = torch.zeros(n_pages_total, n_kv_heads, page_size, D)
        v_pages = torch.zeros_like(k_pages)
        res = []
        rotate = name.endswith("+hadamard")
        for q, k, v, table in seqs:
            if rotate:
                q, k = R.bf16_round(q @ Hn), R.bf16_round(k @ Hn)
            if name.endswith("+rowscale"):
                from . import rowscale as RS
                sc = torch.stack([RS.solve_row_scale(k[:, h]) for h in range(n_kv_heads)])          # [Hkv, D]
                k = R.bf16_round(k * sc[None])
                q = R.bf16_round(q / sc.repeat_interleave(n_q_heads // n_kv_heads, dim=0))
            if name.startswith("e8-"):
                from . import e8_lattice as E8
                kq, vq = E8.quant_dequant(k, "rk4v4"), R.kv_quant_dequant(v, fmt, group)
            else:
                kq, vq = R.kv_quant_dequant(k, fmt, group), R.kv_quant_dequant(v, fmt, group)
            for t in range(k.shape[0]):
                k_pages[table[t // page_size], :, t % page_size] = kq[t]
                v_pages[table[t // page_size], :, t % page_size] = vq[t]
            res.append(paged_decode_reference(q, k_pages, v_pages, table, page_size, k.shape[0]))
        outs[name] = res
        bits = R.kv_bits_per_value(fmt, D, group)
        if name.startswith("e8-"):
            from . import e8_lattice as E8
            bits = (E8.bits_per_value("rk4v4") + bits) / 2          # K on the lattice, V nvfp4
        report["codecs"][name] = {"bits_per_value": bits, "bytes_per_token": 2 * n_kv_heads * D * bits / 8}
    for name in outs:
        errs = [(a - b).abs() for a, b in zip(outs[name], outs["bf16"])]
        report["codecs"][name]["max_abs_err"] = max(float(e.max()) for e in errs)
        report["codecs"][name]["mean_abs_err"] = float(torch.cat([e.flatten() for e in errs]).mean())
    return report


if __name__ == "__main__":
    print(json.dumps(run(), indent=1))
