"""Pure-PyTorch reference of the hybrid decoder (CPU oracle).

Same weights, same math and the same bf16 rounding points as the native
engine, but written with dense per-sequence caches and straight-line torch
ops.  It exists so that greedy parity of the engine can be checked layer by
layer on shrunken configurations without a GPU-side tool.
Math: docs/maintainer/qwen3.6-27b-model.md:112-236 (reference project).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..ops import reference as R
from .config import ModelConfig


def _lin(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x.float() @ w.float().t()


class ReferenceSequence:
    """Holds one sequence's caches: dense K/V per attention layer, conv + ssm state per GDN layer."""

    def __init__(self, cfg: ModelConfig, kv_format: int = R.KV_BF16, int8_group: int = 64, k_hadamard: bool = False):
        self.cfg = cfg
        self.k_hadamard = k_hadamard   # q and k rotated by the normalised Hadamard matrix before k is quantised
        self.kv_format = kv_format
        self.int8_group = int8_group
        self.k: List[torch.Tensor] = [torch.zeros(0, cfg.n_kv_heads, cfg.head_dim) for _ in cfg.attn_layers]
        self.v: List[torch.Tensor] = [torch.zeros(0, cfg.n_kv_heads, cfg.head_dim) for _ in cfg.attn_layers]
        self.conv = [torch.zeros(3, cfg.gdn_conv_dim) for _ in cfg.gdn_layers]
        self.ssm = [torch.zeros(cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.gdn_head_dim) for _ in cfg.gdn_layers]
        self.n_tokens = 0
        # per attention layer (index into cfg.attn_layers): [n_kv_heads, head_dim] channel multipliers of the stored K
        # frame; k is multiplied and q divided, so scores only change through the codec's rounding
        self.k_row_scale: Dict[int, torch.Tensor] = {}


class ReferenceModel:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], prefix: str = "text"):
        self.cfg = cfg
        self.w = {k: v.detach().cpu() for k, v in weights.items()}
        self.prefix = prefix
        # W8A8 / W4A4 engines quantise the GEMM inputs on the fly; set to ops.quant.fake_quant_* to mirror that
        self.act_quant = lambda x: x
        self.rope_inv, self.rope_factor = None, 1.0
        if cfg.rope_yarn_factor > 1.0:
            self.rope_inv, self.rope_factor = R.rope_inv_freq_yarn(cfg.rot_dim, cfg.rope_theta, cfg.rope_yarn_factor,
                                                                   cfg.max_context)

    # ---- pieces ----
    def _attn(self, seq: ReferenceSequence, ai: int, p: str, normed: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        T, D = normed.shape[0], cfg.head_dim
        proj = R.bf16_round(_lin(self.act_quant(normed), self.w[f"{p}/attn/in_proj"]))
        qd, kd = cfg.q_dim, cfg.kv_dim
        q = proj[:, :qd].reshape(T, cfg.n_q_heads, D)
        k = proj[:, qd:qd + kd].reshape(T, cfg.n_kv_heads, D)
        gate = proj[:, qd + kd: 2 * qd + kd]
        v = proj[:, 2 * qd + kd:].reshape(T, cfg.n_kv_heads, D)
        q = R.bf16_round(R.rmsnorm(q, self.w[f"{p}/attn/q_norm"], cfg.rms_eps, True))
        k = R.bf16_round(R.rmsnorm(k, self.w[f"{p}/attn/k_norm"], cfg.rms_eps, True))
        q = R.bf16_round(R.rope_partial(q, pos, cfg.rot_dim, cfg.rope_theta, self.rope_factor, self.rope_inv))
        k = R.rope_partial(k, pos, cfg.rot_dim, cfg.rope_theta, self.rope_factor, self.rope_inv)
        if seq.k_hadamard:
            Hn = R.hadamard_matrix(D)
            q = R.bf16_round(q @ Hn)
            k = k @ Hn
        rs = seq.k_row_scale.get(ai)
        if rs is not None:
            rs = R.bf16_round(rs.float())
            k = k * rs[None]
            q = R.bf16_round(q / rs.repeat_interleave(cfg.n_q_heads // cfg.n_kv_heads, dim=0)[None])
        k = R.kv_quant_dequant(k, seq.kv_format, seq.int8_group)
        v = R.kv_quant_dequant(v, seq.kv_format, seq.int8_group)
        base = seq.k[ai].shape[0]
        seq.k[ai] = torch.cat([seq.k[ai], k], 0)
        seq.v[ai] = torch.cat([seq.v[ai], v], 0)
        kv_len = base + torch.arange(T) + 1
        o = R.gqa_attention(q, seq.k[ai], seq.v[ai], kv_len, 1.0 / math.sqrt(D))
        o = R.bf16_round(o).reshape(T, qd)
        return R.bf16_round(o * torch.sigmoid(gate))

    def _gdn(self, seq: ReferenceSequence, gi: int, p: str, normed: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        T, d = normed.shape[0], cfg.gdn_head_dim
        proj = R.bf16_round(_lin(self.act_quant(normed), self.w[f"{p}/gdn/in_proj"]))
        C, vd, hv = cfg.gdn_conv_dim, cfg.gdn_v_dim, cfg.gdn_v_heads
        conv, seq.conv[gi] = R.causal_conv1d_silu(proj[:, :C], self.w[f"{p}/gdn/conv_w"], seq.conv[gi])
        conv = R.bf16_round(conv)
        qk = cfg.gdn_qk_dim
        q = conv[:, :qk].reshape(T, cfg.gdn_qk_heads, d)
        k = conv[:, qk:2 * qk].reshape(T, cfg.gdn_qk_heads, d)
        v = conv[:, 2 * qk:].reshape(T, hv, d)
        z = proj[:, C:C + vd].reshape(T, hv, d)
        a, b = proj[:, C + vd:C + vd + hv], proj[:, C + vd + hv:C + vd + 2 * hv]
        g, beta = R.gdn_gating(a, b, self.w[f"{p}/gdn/A_log"], self.w[f"{p}/gdn/dt_bias"])
        o, seq.ssm[gi] = R.gdn_recurrent(q, k, v, g, beta, seq.ssm[gi])
        o = R.bf16_round(o)
        y = R.gated_rmsnorm(o, z, self.w[f"{p}/gdn/norm"], cfg.rms_eps)
        return R.bf16_round(y).reshape(T, vd)

    def _ffn(self, p: str, normed: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if cfg.moe is None:
            gu = _lin(self.act_quant(normed), self.w[f"{p}/mlp/gate_up"])
            i = gu.shape[1] // 2
            act = R.bf16_round(torch.nn.functional.silu(gu[:, :i]) * gu[:, i:])
            return _lin(self.act_quant(act), self.w[f"{p}/mlp/down"])
        m = cfg.moe
        router = R.bf16_round(_lin(normed, self.w[f"{p}/moe/router"]))  # logits are a bf16 op boundary
        wts, ids = R.moe_route(router[:, : m.n_experts], m.top_k, m.norm_topk)
        out = torch.zeros(normed.shape[0], cfg.hidden)
        gu_all, dn_all = self.w[f"{p}/moe/experts_gate_up"], self.w[f"{p}/moe/experts_down"]
        for t in range(normed.shape[0]):
            for j in range(m.top_k):
                e = int(ids[t, j])
                gu = _lin(normed[t:t + 1], gu_all[e])
                act = R.bf16_round(torch.nn.functional.silu(gu[:, : m.expert_inter]) * gu[:, m.expert_inter:])
                out[t] += wts[t, j] * _lin(act, dn_all[e])[0]
        gu = _lin(normed, self.w[f"{p}/moe/shared_gate_up"])
        act = R.bf16_round(torch.nn.functional.silu(gu[:, : m.shared_inter]) * gu[:, m.shared_inter:])
        shared = _lin(act, self.w[f"{p}/moe/shared_down"])
        return out + torch.sigmoid(router[:, m.n_experts:]) * shared

    # ---- forward over T new tokens of one sequence ----
    def forward(self, seq: ReferenceSequence, ids: torch.Tensor, trace: Optional[dict] = None,
                positions: Optional[torch.Tensor] = None, embed_rows: Optional[torch.Tensor] = None,
                embed_vals: Optional[torch.Tensor] = None, layers: Optional[tuple] = None,
                hidden_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`positions` ([T] or [T, 3]) overrides the default cache positions for the rope; `embed_vals` rows replace the
        token embeddings at `embed_rows` (visual tokens of a multimodal prompt).

        Pipeline stages: `layers = (first, end)` runs only that half-open range of layers; a stage that does not start
        at layer 0 takes the residual stream of the previous stage as `hidden_in` [T, hidden], and a stage that does
        not end at the last layer returns the residual stream instead of the final-normed hidden states.  The token
        count of the sequence advances on the last stage only."""
        cfg, pf = self.cfg, self.prefix
        T = ids.shape[0]
        first, end = layers if layers is not None else (0, cfg.n_layers)
        pos = seq.n_tokens + torch.arange(T) if positions is None else positions
        if first == 0:
            x = self.w[f"{pf}/embed"][ids.long()].float()
            if embed_rows is not None:
                x[embed_rows.long()] = embed_vals.float()
        else:
            x = R.bf16_round(hidden_in.float())
        for layer in range(first, end):
            p = f"{pf}/layers/{layer}"
            normed = R.bf16_round(R.rmsnorm(x, self.w[f"{p}/input_norm"], cfg.rms_eps, True))
            if cfg.is_full_attn(layer):
                mix = self._attn(seq, cfg.attn_layers.index(layer), p, normed, pos)
                w_out = self.w[f"{p}/attn/o_proj"]
            else:
                mix = self._gdn(seq, cfg.gdn_layers.index(layer), p, normed)
                w_out = self.w[f"{p}/gdn/out_proj"]
            x = R.bf16_round(x + _lin(self.act_quant(mix), w_out))
            normed = R.bf16_round(R.rmsnorm(x, self.w[f"{p}/post_norm"], cfg.rms_eps, True))
            x = R.bf16_round(x + self._ffn(p, normed))
            if trace is not None:
                trace[f"layer{layer}"] = x.clone()
        if end < cfg.n_layers:
            return x
        seq.n_tokens += T
        hidden = R.bf16_round(R.rmsnorm(x, self.w[f"{pf}/final_norm"], cfg.rms_eps, True))
        if trace is not None:
            trace["final"] = hidden.clone()
        return hidden

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return R.bf16_round(_lin(self.act_quant(hidden), self.w[f"{self.prefix}/lm_head"]))

    def generate_greedy(self, prompt: torch.Tensor, n_new: int, kv_format: int = R.KV_BF16) -> List[int]:
        seq = ReferenceSequence(self.cfg, kv_format)
        h = self.forward(seq, prompt)
        out = []
        tok = int(R.argmax_lowest(self.logits(h[-1:]))[0])
        out.append(tok)
        for _ in range(n_new - 1):
            h = self.forward(seq, torch.tensor([tok]))
            tok = int(R.argmax_lowest(self.logits(h))[0])
            out.append(tok)
        return out
