"""DFlash: a block-diffusion draft model that proposes a whole block of tokens in ONE pass.

The target model exports the residual stream of a few of its layers ("features") for every committed token.  The
draft model keeps, per draft layer, a KV cache of the *context*: keys and values projected from those features
(`feature_proj` -> RMSNorm -> per-layer `ctx_kv`, key norm, RoPE).  To propose, it embeds a block
`[anchor token, MASK, ..., MASK]` of K positions at the frontier, runs its few decoder layers over the block -- every
block position attends to the context keys AND to every other position of the block (no causal mask inside the block:
that is what makes it a denoising step instead of K sequential steps) -- and reads K tokens off the shared LM head:
row i predicts the token after position frontier + i.  The target then verifies the K proposals in its usual single
pass, and the features of the accepted positions are appended to the context caches.

This follows the reference's DFlash drafter in function: context append and proposal in
src/targets/qwen3_6/impl/runtime/dflash_impl.h:98-551 (feature projection + context norm, per-layer context K / V,
`prepare_masked_block`, bidirectional block attention over a cached context, shared embedding and LM head), with a
sliding-window ("local") context for the first layers (src/core/cyclic_kv_cache.h, ops::swa) and a full context for
the rest.  The decoder block itself is this repository's gated-attention block, so the proposal pass runs on the same
kernels as the target (models/hybrid.py); only the context append is specific.

`DFlashReference` is the dense fp32 oracle of both steps; `runtime/dflash.py` is the native path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Dict, List, Sequence

import torch

from ..ops import reference as R
from .config import ModelConfig
from .weights import random_weights


@dataclass(frozen=True)
class DFlashConfig:
    n_layers: int = 2              # draft decoder layers
    local_layers: int = 1          # the first `local_layers` see only the last `window` context tokens
    window: int = 256              # context window of the local layers (0: every layer sees the whole context)
    feature_layers: tuple = ()     # target layers whose residual stream is a feature block (default: middle and last)
    ffn_inter: int = 0             # draft MLP width (default: the target's)
    mask_token: int = 0            # id embedded at the not-yet-known block positions

    def resolved(self, target: ModelConfig) -> "DFlashConfig":
        fl = self.feature_layers or tuple(sorted({target.n_layers // 2 - 1 if target.n_layers > 1 else 0,
                                                  target.n_layers - 1}))
        return replace(self, feature_layers=fl, ffn_inter=self.ffn_inter or target.ffn_inter,
                       local_layers=min(self.local_layers, self.n_layers) if self.window > 0 else 0)


def draft_model_config(target: ModelConfig, dc: DFlashConfig) -> ModelConfig:
    """The draft decoder as a ModelConfig: `n_layers` gated full-attention layers with the target's head geometry."""
    dense = replace(target, moe=None) if target.moe is not None else target
    return replace(dense, name=f"{target.name}-dflash", n_layers=dc.n_layers, full_attn_interval=1,
                   ffn_inter=dc.ffn_inter or target.ffn_inter or 4 * target.hidden, mtp_layers=0)


def random_dflash_weights(target: ModelConfig, dc: DFlashConfig, target_weights: Dict[str, torch.Tensor], device,
                          seed: int = 7, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random-init draft weights under the prefix `dflash/`; embedding and LM head are the target's tensors."""
    dc = dc.resolved(target)
    cfg = draft_model_config(target, dc)
    base = random_weights(cfg, device, seed=seed, std=std)
    out: Dict[str, torch.Tensor] = {}
    for k, v in base.items():
        if k in ("text/embed", "text/lm_head"):
            continue
        out["dflash/" + k.split("/", 1)[1]] = v
    out["dflash/embed"] = target_weights["text/embed"]
    out["dflash/lm_head"] = target_weights["text/lm_head"]
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 1)
    h, F = target.hidden, len(dc.feature_layers)

    def rnd(*shape, s=std):
        t = torch.empty(shape, dtype=torch.bfloat16, device=device)
        t.normal_(0.0, s, generator=gen)
        return t
    out["dflash/feature_proj"] = rnd(h, F * h, s=std / math.sqrt(F))
    out["dflash/context_norm"] = rnd(h)
    for l in range(dc.n_layers):
        out[f"dflash/layers/{l}/ctx_kv"] = rnd(2 * cfg.kv_dim, h)   # rows: context keys, then context values
    return out


class DFlashReference:
    """Dense fp32 oracle (CPU): one instance per sequence."""

    def __init__(self, target: ModelConfig, dc: DFlashConfig, weights: Dict[str, torch.Tensor]):
        self.dc = dc.resolved(target)
        self.cfg = draft_model_config(target, self.dc)
        self.w = {k: v.detach().float().cpu() for k, v in weights.items() if k.startswith("dflash/")}
        cfg = self.cfg
        self.k: List[torch.Tensor] = [torch.zeros(0, cfg.n_kv_heads, cfg.head_dim) for _ in range(cfg.n_layers)]
        self.v: List[torch.Tensor] = [torch.zeros(0, cfg.n_kv_heads, cfg.head_dim) for _ in range(cfg.n_layers)]

    @property
    def n_context(self) -> int:
        return self.k[0].shape[0]

    def append_context(self, features: torch.Tensor) -> None:
        """features [n, F * hidden]: the tapped residual streams of the next n committed positions."""
        cfg, n0 = self.cfg, self.n_context
        f = R.bf16_round(features.float())
        c = R.bf16_round(f @ self.w["dflash/feature_proj"].t())
        c = R.bf16_round(R.rmsnorm(c, self.w["dflash/context_norm"], cfg.rms_eps, True))
        pos = torch.arange(n0, n0 + f.shape[0])
        for l in range(cfg.n_layers):
            kv = R.bf16_round(c @ self.w[f"dflash/layers/{l}/ctx_kv"].t())
            k = kv[:, : cfg.kv_dim].reshape(-1, cfg.n_kv_heads, cfg.head_dim)
            v = kv[:, cfg.kv_dim:].reshape(-1, cfg.n_kv_heads, cfg.head_dim)
            k = R.bf16_round(R.rmsnorm(k, self.w[f"dflash/layers/{l}/attn/k_norm"], cfg.rms_eps, True))
            k = R.bf16_round(R.rope_partial(k, pos, cfg.rot_dim, cfg.rope_theta))
            self.k[l] = torch.cat([self.k[l], k], 0)
            self.v[l] = torch.cat([self.v[l], v], 0)

    def logits(self, anchor: int, K: int) -> torch.Tensor:
        """[K, vocab] logits of the block [anchor, MASK x (K - 1)] placed at the frontier (= context length)."""
        cfg, dc, w = self.cfg, self.dc, self.w
        n, D = self.n_context, cfg.head_dim
        ids = torch.tensor([anchor] + [dc.mask_token] * (K - 1))
        pos = torch.arange(n, n + K)
        x = w["dflash/embed"][ids]
        for l in range(cfg.n_layers):
            p = f"dflash/layers/{l}"
            normed = R.bf16_round(R.rmsnorm(x, w[f"{p}/input_norm"], cfg.rms_eps, True))
            proj = R.bf16_round(normed @ w[f"{p}/attn/in_proj"].t())
            qd, kd = cfg.q_dim, cfg.kv_dim
            q = proj[:, :qd].reshape(K, cfg.n_q_heads, D)
            k = proj[:, qd:qd + kd].reshape(K, cfg.n_kv_heads, D)
            gate = proj[:, qd + kd:2 * qd + kd]
            v = proj[:, 2 * qd + kd:].reshape(K, cfg.n_kv_heads, D)
            q = R.bf16_round(R.rmsnorm(q, w[f"{p}/attn/q_norm"], cfg.rms_eps, True))
            k = R.bf16_round(R.rmsnorm(k, w[f"{p}/attn/k_norm"], cfg.rms_eps, True))
            q = R.bf16_round(R.rope_partial(q, pos, cfg.rot_dim, cfg.rope_theta))
            k = R.bf16_round(R.rope_partial(k, pos, cfg.rot_dim, cfg.rope_theta))
            keys = torch.cat([self.k[l], k], 0)
            vals = torch.cat([self.v[l], R.bf16_round(v)], 0)
            vis = torch.ones(K, n + K, dtype=torch.bool)          # the block is bidirectional
            if l < dc.local_layers:
                # a local layer sees the last `window` keys of its own causal horizon, like a sliding-window
                # attention whose horizon ends at the block's last position
                vis[:, : max(0, n + K - dc.window)] = False
            o = R.gqa_attention(q, keys, vals, None, 1.0 / math.sqrt(D), vis)
            o = R.bf16_round(R.bf16_round(o).reshape(K, qd) * torch.sigmoid(gate))
            x = R.bf16_round(x + o @ w[f"{p}/attn/o_proj"].t())
            normed = R.bf16_round(R.rmsnorm(x, w[f"{p}/post_norm"], cfg.rms_eps, True))
            gu = normed @ w[f"{p}/mlp/gate_up"].t()
            i = gu.shape[1] // 2
            act = R.bf16_round(torch.nn.functional.silu(gu[:, :i]) * gu[:, i:])
            x = R.bf16_round(x + act @ w[f"{p}/mlp/down"].t())
        hid = R.bf16_round(R.rmsnorm(x, w["dflash/final_norm"], cfg.rms_eps, True))
        return R.bf16_round(hid @ w["dflash/lm_head"].t())

    def propose(self, anchor: int, K: int) -> List[int]:
        return [int(t) for t in self.logits(anchor, K).argmax(-1)]


def reference_features(hidden_by_layer: Sequence[torch.Tensor]) -> torch.Tensor:
    """Concatenates the tapped residual streams ([n, hidden] each) into the feature rows [n, F * hidden]."""
    return torch.cat([h.float() for h in hidden_by_layer], dim=-1)
