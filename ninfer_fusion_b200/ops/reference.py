"""Plain-PyTorch fp32 oracles of every kernel's math.

These run on CPU and are the numerics baseline for the CUDA kernels: independent
oracles at small exhaustive shapes are the safety net where no memory checker
runs.  Contracts follow the
reference's operator headers (include/ninfer/ops/*.h); bf16 rounding points
are placed where an operator boundary stores bf16.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

E2M1_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])

KV_BF16, KV_FP8_ROW, KV_INT8_GROUP, KV_NVFP4 = 0, 1, 2, 3
KV_FORMAT_NAMES = {"bf16": KV_BF16, "fp8": KV_FP8_ROW, "int8": KV_INT8_GROUP, "nvfp4": KV_NVFP4}


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, unit_offset: bool = True) -> torch.Tensor:
    x = x.float()
    wf = w.float() + (1.0 if unit_offset else 0.0)
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * wf


def rope_inv_freq(rot_dim: int, theta: float) -> torch.Tensor:
    half = rot_dim // 2
    return (theta ** (-torch.arange(half, dtype=torch.float64) / half)).float()


def rope_inv_freq_yarn(rot_dim: int, theta: float, factor: float = 4.0, original_context: int = 262144,
                       beta_fast: float = 32.0, beta_slow: float = 1.0):
    """YaRN frequency table and attention factor (reference: yarn4, include/ninfer/ops/rope.h:110-117).

    Pairs that rotate more than `beta_fast` times over the original context keep their frequency, pairs that
    rotate less than `beta_slow` times are interpolated by `factor`, the band in between is blended linearly.
    The returned factor 0.1 * ln(factor) + 1 (1.1386 for x4) multiplies cos and sin."""
    half = rot_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) / half)

    def dim_of(rotations: float) -> float:
        return (rot_dim * math.log(original_context / (rotations * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(dim_of(beta_fast)), 0)
    high = min(math.ceil(dim_of(beta_slow)), half - 1)
    ramp = ((torch.arange(half, dtype=torch.float64) - low) / max(high - low, 1e-3)).clamp(0, 1)
    keep = 1.0 - ramp                       # 1 = extrapolate (original frequency), 0 = interpolate
    out = inv / factor * (1 - keep) + inv * keep
    return out.float(), 0.1 * math.log(factor) + 1.0


def hadamard_matrix(n: int) -> torch.Tensor:
    """Normalised Sylvester-Hadamard matrix (symmetric, orthogonal): H_n / sqrt(n), n a power of two."""
    H = torch.ones(1, 1)
    while H.shape[0] < n:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return H / math.sqrt(n)


def rope_partial(x: torch.Tensor, pos: torch.Tensor, rot_dim: int, theta: float,
                 attn_factor: float = 1.0, inv_freq: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, H, D]; NeoX split-half rotation on the first rot_dim dims.

    pos is [T] or [T, 3] (MRoPE: rotary pair i uses axis i % 3)."""
    x = x.float()
    half = rot_dim // 2
    inv = (rope_inv_freq(rot_dim, theta) if inv_freq is None else inv_freq).to(x.device)
    if pos.dim() == 1:
        p = pos.float()[:, None].expand(-1, half)
    else:
        axis = torch.arange(half, device=x.device) % 3
        p = pos.float()[:, axis]
    ang = p * inv[None, :]
    cs, sn = torch.cos(ang)[:, None, :] * attn_factor, torch.sin(ang)[:, None, :] * attn_factor
    x1, x2 = x[..., :half], x[..., half:rot_dim]
    out = x.clone()
    out[..., :half] = x1 * cs - x2 * sn
    out[..., half:rot_dim] = x2 * cs + x1 * sn
    return out


# ----------------------------------------------------------------------------
# KV codecs: quantise -> (codes, scales) as float tensors of representable values
# ----------------------------------------------------------------------------
def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).to(torch.float32)


def e2m1_round(x: torch.Tensor) -> torch.Tensor:
    """Round to nearest (ties to even code) on the e2m1 grid, saturating at 6."""
    a = x.abs()
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
    # ties go to the even mantissa: .25->0, .75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4, 5->4
    up_on_tie = torch.tensor([False, True, False, True, False, True, False], device=x.device)
    idx = torch.zeros_like(a, dtype=torch.long)
    for b, up in zip(bounds, up_on_tie):
        idx += (a >= b).long() if up else (a > b).long()
    return torch.sign(x) * E2M1_GRID.to(x.device)[idx]


def kv_quant_dequant(x: torch.Tensor, fmt: int, group: int = 64, bf16_input: bool = True) -> torch.Tensor:
    """What an attention kernel sees after a row [.., D] went through the cache codec.  `bf16_input=False`: the row
    is already the fp32 decode of another codec (a cell re-encoded from one tier to the next) and is taken as is."""
    x = bf16_round(x.float()) if bf16_input else x.float()
    if fmt == KV_BF16:
        return x
    if fmt == KV_FP8_ROW:
        amax = x.abs().amax(-1, keepdim=True)
        s = (amax / 448.0).clamp(2.0 ** -24, 65504.0).to(torch.float16).float()
        return e4m3_round(x / s) * s
    if fmt == KV_INT8_GROUP:
        g = x.reshape(*x.shape[:-1], -1, group)
        s = (g.abs().amax(-1, keepdim=True) / 127.0).to(torch.float16).float()
        q = torch.where(s > 0, torch.round(g / torch.where(s > 0, s, torch.ones_like(s))), torch.zeros_like(g))
        q = q.clamp(-127, 127)
        return (q * s).reshape(x.shape)
    if fmt == KV_NVFP4:
        g = x.reshape(*x.shape[:-1], -1, 16)
        s = e4m3_round(g.abs().amax(-1, keepdim=True) / 6.0)
        q = torch.where(s > 0, g / torch.where(s > 0, s, torch.ones_like(s)), torch.zeros_like(g))
        return (e2m1_round(q) * s).reshape(x.shape)
    raise ValueError(f"unknown KV format {fmt}")


def kv_bits_per_value(fmt: int, head_dim: int = 256, group: int = 64) -> float:
    if fmt == KV_BF16:
        return 16.0
    if fmt == KV_FP8_ROW:
        return 8.0 + 16.0 / head_dim
    if fmt == KV_INT8_GROUP:
        return 8.0 + 16.0 / group
    return 4.0 + 8.0 / 16


def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_len: torch.Tensor | None = None,
                  scale: float | None = None, mask: torch.Tensor | None = None) -> torch.Tensor:
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] (already dequantised).  Query i sees keys < kv_len[i]
    (and mask[i, j] if given).  Returns [Tq, Hq, D] fp32."""
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    kk = k.float().repeat_interleave(g, dim=1)
    vv = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    vis = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device)
    if kv_len is not None:
        vis &= torch.arange(Tk, device=q.device)[None, :] < kv_len[:, None]
    if mask is not None:
        vis &= mask
    s = s.masked_fill(~vis[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("hqk,khd->qhd", p, vv)


def selected_block_mask(kv_len: torch.Tensor, sel_blocks: torch.Tensor, sel_count: torch.Tensor, n_keys: int) -> torch.Tensor:
    """Visibility of selected-block attention: query i sees the 4-token blocks sel_blocks[i, :sel_count[i]] and the
    tokens of its incomplete last block [4 * (kv_len // 4), kv_len).  Returns bool [Tq, n_keys] for gqa_attention."""
    Tq = kv_len.numel()
    vis = torch.zeros((Tq, n_keys), dtype=torch.bool)
    for i in range(Tq):
        n = int(kv_len[i])
        for b in sel_blocks[i, : int(sel_count[i])].tolist():
            vis[i, 4 * b: 4 * b + 4] = True
        vis[i, (n // 4) * 4: n] = True
    return vis


# ----------------------------------------------------------------------------
# Gated DeltaNet
# ----------------------------------------------------------------------------
def causal_conv1d_silu(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x [T, C] one sequence, w [C, 4] (tap 3 = newest), state [3, C] oldest->newest.
    Returns (silu(conv) [T, C] fp32, new state [3, C])."""
    xf = torch.cat([state.float(), x.float()], dim=0)  # [T+3, C]
    T = x.shape[0]
    acc = torch.zeros(T, x.shape[1], device=x.device)
    for j in range(4):
        acc += w.float()[:, j][None, :] * xf[j:j + T]
    return torch.nn.functional.silu(acc), xf[-3:].clone()


def gdn_gating(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    g = -torch.exp(A_log.float()) * torch.nn.functional.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


def gdn_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                  state: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """One sequence.  q,k [T, Hk, 128], v [T, Hv, 128], g,beta [T, Hv], state [Hv, dv, dk] fp32.
    Returns (o [T, Hv, dv], new state)."""
    T, Hk, dk = q.shape
    Hv = v.shape[1]
    rep = Hv // Hk
    qn = q.float() * torch.rsqrt(q.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    kn = k.float() * torch.rsqrt(k.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    qn = qn.repeat_interleave(rep, dim=1) / math.sqrt(dk)
    kn = kn.repeat_interleave(rep, dim=1)
    S = state.double().clone()
    out = torch.zeros(T, Hv, v.shape[-1], dtype=torch.float64, device=q.device)
    for t in range(T):
        alpha = torch.exp(g[t].double())[:, None, None]
        S = S * alpha
        kt = kn[t].double()
        u = beta[t].double()[:, None] * (v[t].double() - torch.einsum("hvk,hk->hv", S, kt))
        S = S + u[:, :, None] * kt[:, None, :]
        out[t] = torch.einsum("hvk,hk->hv", S, qn[t].double())
    return out.float(), S.float()


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    o = o.float()
    return o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * w.float() * torch.nn.functional.silu(z.float())


# ----------------------------------------------------------------------------
# MoE routing
# ----------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, top_k: int, renorm: bool = True):
    """softmax over experts -> top-k (ties: lower id) -> renormalise.  Returns (weights, ids)."""
    p = torch.softmax(logits.float(), dim=-1)
    # stable descending sort keeps the lower id first among equal probabilities
    vals, idx = torch.sort(p, dim=-1, descending=True, stable=True)
    vals, idx = vals[..., :top_k], idx[..., :top_k]
    if renorm:
        vals = vals / vals.sum(-1, keepdim=True)
    return vals, idx


# ----------------------------------------------------------------------------
# Sampling / speculative acceptance
# ----------------------------------------------------------------------------
def argmax_lowest(logits: torch.Tensor) -> torch.Tensor:
    m = logits.float().amax(-1, keepdim=True)
    V = logits.shape[-1]
    idx = torch.arange(V, device=logits.device).expand_as(logits)
    return torch.where(logits.float() == m, idx, torch.full_like(idx, V)).amin(-1).int()


def accept_greedy_chain(target: torch.Tensor, draft: torch.Tensor):
    """target [B, K+1], draft [B, K] -> (n_accepted [B], out_tokens [B, K+1] padded with -1)."""
    B, K = draft.shape
    n_acc = torch.zeros(B, dtype=torch.int32)
    out = torch.full((B, K + 1), -1, dtype=torch.int32)
    for b in range(B):
        n = 0
        while n < K and int(draft[b, n]) == int(target[b, n]):
            n += 1
        n_acc[b] = n
        out[b, :n] = draft[b, :n]
        out[b, n] = target[b, n]
    return n_acc, out


def accept_greedy_tree(target: torch.Tensor, tok: torch.Tensor, parent: torch.Tensor, max_depth: int):
    B, N = tok.shape
    n_acc = torch.zeros(B, dtype=torch.int32)
    out_t = torch.full((B, max_depth + 1), -1, dtype=torch.int32)
    out_n = torch.full((B, max_depth + 1), -1, dtype=torch.int32)
    for b in range(B):
        acc, depth = [True] + [False] * (N - 1), [0] * N
        best, best_d = 0, 0
        for i in range(1, N):
            p = int(parent[b, i])
            ok = 0 <= p < i
            acc[i] = ok and acc[p] and int(tok[b, i]) == int(target[b, p])
            depth[i] = depth[p] + 1 if ok else 0
            if acc[i] and depth[i] > best_d:
                best, best_d = i, depth[i]
        n_acc[b] = best_d
        node = best
        for d in range(best_d, 0, -1):
            out_t[b, d - 1] = tok[b, node]
            out_n[b, d - 1] = node
            node = int(parent[b, node])
        out_t[b, best_d] = target[b, best]
        out_n[b, best_d] = best
    return n_acc, out_t, out_n
