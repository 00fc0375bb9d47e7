"""KVarN k4v2 tile codec (oracle): 128-token tiles, K at 4 bits and V at 2 bits with two-sided scaling.

A tile is [G = 128 tokens, D channels].  K is first balanced by `iterations` rounds of alternating normalisation
(divide every token row by its RMS, then every channel column by its RMS; the accumulated token and channel factors are
kept), then quantised to 4-bit codes with one fp16 (scale, zero) pair per channel over the tile's tokens.  V is
balanced the same way and quantised to 2-bit codes with one fp16 (scale, zero) pair per token over the channels.  The
first `sink` tokens of a sequence and the tokens after the last complete tile stay bf16 (sink page and tail slots).

Record of one tile at D = 256: 16384 B K codes + 512 B channel scales + 512 B channel zeros + 256 B token scales, then
8192 B V codes + 512 B channel scales + 256 B token scales + 256 B token zeros = 26880 bytes, 3.28 bits per value.
Reference: include/ninfer/ops/kvarn.h (kvarn_k4v2_g128 profile, record offsets, 8 iterations, 1 sink page, 3 tail
slots); that op family is not wired into the reference's build either, and no kernel here reads this format.
"""
from __future__ import annotations

import torch

GROUP = 128
ITERATIONS = 8


def record_bytes(head_dim: int = 256, group: int = GROUP) -> int:
    k = group * head_dim // 2 + 2 * head_dim + 2 * head_dim + 2 * group
    v = group * head_dim // 4 + 2 * head_dim + 2 * group + 2 * group
    return k + v


def bits_per_value(head_dim: int = 256, group: int = GROUP) -> float:
    return record_bytes(head_dim, group) * 8 / (2 * group * head_dim)


def _balance(x: torch.Tensor, iterations: int):
    """x [G, D] -> (balanced x, token factors [G, 1], channel factors [1, D]) with x = balanced * token * channel."""
    tok = torch.ones((x.shape[0], 1))
    ch = torch.ones((1, x.shape[1]))
    y = x.clone()
    for _ in range(iterations):
        r = y.pow(2).mean(1, keepdim=True).sqrt().clamp_min(1e-8)
        y, tok = y / r, tok * r
        c = y.pow(2).mean(0, keepdim=True).sqrt().clamp_min(1e-8)
        y, ch = y / c, ch * c
    return y, tok.to(torch.float16).float(), ch.to(torch.float16).float()


def _asym(y: torch.Tensor, levels: int, dim: int) -> torch.Tensor:
    """Asymmetric uniform quantiser along `dim`: fp16 scale and zero, codes 0 .. levels - 1; returns the value map."""
    lo, hi = y.amin(dim, keepdim=True), y.amax(dim, keepdim=True)
    scale = ((hi - lo) / (levels - 1)).to(torch.float16).float()
    zero = lo.to(torch.float16).float()
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    code = torch.clamp(torch.round((y - zero) / safe), 0, levels - 1)
    return torch.where(scale > 0, code * scale + zero, zero.expand_as(y))


def quant_dequant_tile(k: torch.Tensor, v: torch.Tensor, iterations: int = ITERATIONS):
    """One complete tile: k, v [G, D] fp32 -> what attention sees after the codec."""
    yk, tk, ck = _balance(k.float(), iterations)
    # the channel factor of K folds into the per-channel (scale, zero) pair; the token factor is stored beside it
    kq = _asym(yk * ck, 16, dim=0) * tk
    yv, tv, cv = _balance(v.float(), iterations)
    vq = _asym(yv * tv, 4, dim=1) * cv
    return kq, vq


def quant_dequant_sequence(k: torch.Tensor, v: torch.Tensor, sink: int = 16, group: int = GROUP):
    """k, v [n, Hkv, D]: sink tokens and the incomplete last tile stay as they are (bf16 storage), complete tiles after
    the sink go through the tile codec per KV head."""
    n, H, _ = k.shape
    kq, vq = k.clone().float(), v.clone().float()
    start = min(sink, n)
    while start + group <= n:
        for h in range(H):
            a, b = quant_dequant_tile(k[start:start + group, h], v[start:start + group, h])
            kq[start:start + group, h], vq[start:start + group, h] = a, b
        start += group
    return kq, vq
