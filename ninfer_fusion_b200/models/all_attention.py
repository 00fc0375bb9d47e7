"""fp32 oracle runtime of the all-attention packages (sliding-window / full / NoPE layer schedules).

The hybrid GDN family is served by the GPU runtime; the packages described in `models/packages.py` whose schedule is
attention only (Spark-X2.5-4B, Muse-Glimmer-30B, Gemma-4-31B) run here, on the CPU, through the same Program API as
every other model: one decoder class driven entirely by the package description --

* per layer: FULL or SLIDING (the last `window` keys of the causal horizon), its own head counts and head width, its
  own rotary width (0 = no positional rotation) and base;
* optional q / k RMS norm, an optional learned-constant factor on q . k, optional K shared with V on full layers;
* optional head-wise output gate (one sigmoid gate per query head);
* pre-norm residual branches, optionally with a second norm on each branch's OUTPUT before it is added;
* SwiGLU or GeGLU (exact or tanh) feed-forward;
* tied or separate LM head, an output multiplier, final logit soft-capping `cap * tanh(logits / cap)`.

The GPU runtime still refuses these packages by naming the capabilities it lacks; this file is the reference their
kernels will be tested against and the path `--device cpu` serves them on.

Reference: src/targets/{spark_x2_5_4b,muse_glimmer_30b,gemma4_31b}/impl/config.h (geometry, schedules, soft-capping,
NoPE layers, head-wise gate, K = V), src/targets/registry.cpp (one Program API for every package).
"""
from __future__ import annotations

import math
from dataclasses import replace
from typing import Dict, List, Optional

import torch

from ..ops import reference as R
from .config import ModelConfig
from .packages import FULL, SLIDING, LayerKind, Package


def shrink_package(pkg: Package, n_layers: int, vocab: Optional[int] = None, hidden_div: int = 1) -> Package:
    """The first `n_layers` of the package's schedule (debug / test geometry); optionally a smaller vocabulary and all
    widths divided by `hidden_div` (head widths stay, head counts shrink)."""
    def shrink_layer(l: LayerKind) -> LayerKind:
        return replace(l, q_heads=max(1, l.q_heads // hidden_div), kv_heads=max(1, l.kv_heads // hidden_div))
    return replace(pkg, model_id=f"{pkg.model_id}@{n_layers}", n_layers=n_layers,
                   layers=tuple(shrink_layer(l) for l in pkg.layers[:n_layers]), hidden=pkg.hidden // hidden_div,
                   intermediate=pkg.intermediate // hidden_div, vocab=vocab or pkg.vocab)


def package_traits(pkg: Package) -> Dict[str, object]:
    n = pkg.needs
    return {"qk_norm": "qk-norm" in n, "headwise_gate": "headwise-attention-gate" in n,
            "post_branch_norms": "post-branch-norms" in n, "k_equals_v": "k-equals-v" in n,
            "geglu": "geglu-mlp" in n, "gelu_tanh": pkg.activation == "gelu_pytorch_tanh",
            "qk_scale": float(getattr(pkg, "qk_scale", 1.0)), "output_multiplier": float(getattr(pkg, "output_multiplier", 1.0))}


def random_package_weights(pkg: Package, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    t = package_traits(pkg)

    def rnd(*shape, s=std):
        return torch.randn(shape, generator=g) * s
    h = pkg.hidden
    w: Dict[str, torch.Tensor] = {"text/embed": rnd(pkg.vocab, h), "text/final_norm": rnd(h, s=0.02)}
    if not pkg.tie_word_embeddings:
        w["text/lm_head"] = rnd(pkg.vocab, h)
    for i, l in enumerate(pkg.layers):
        p = f"text/layers/{i}"
        qd, kd = l.q_heads * l.head_dim, l.kv_heads * l.head_dim
        w[f"{p}/input_norm"], w[f"{p}/post_norm"] = rnd(h, s=0.02), rnd(h, s=0.02)
        w[f"{p}/attn/q_proj"], w[f"{p}/attn/k_proj"], w[f"{p}/attn/o_proj"] = rnd(qd, h), rnd(kd, h), rnd(h, qd)
        if not (t["k_equals_v"] and l.kind == FULL):
            w[f"{p}/attn/v_proj"] = rnd(kd, h)
        if t["qk_norm"]:
            w[f"{p}/attn/q_norm"], w[f"{p}/attn/k_norm"] = rnd(l.head_dim, s=0.02), rnd(l.head_dim, s=0.02)
        if t["headwise_gate"]:
            w[f"{p}/attn/gate"] = rnd(l.q_heads, h)
        if t["post_branch_norms"]:
            w[f"{p}/attn_out_norm"], w[f"{p}/mlp_out_norm"] = rnd(h, s=0.02), rnd(h, s=0.02)
        w[f"{p}/mlp/gate_up"], w[f"{p}/mlp/down"] = rnd(2 * pkg.intermediate, h), rnd(h, pkg.intermediate)
    return w


class PackageSequence:
    """One sequence's caches: dense K / V per layer (each layer has its own head geometry)."""

    def __init__(self, pkg: Package):
        self.k: List[torch.Tensor] = [torch.zeros(0, l.kv_heads, l.head_dim) for l in pkg.layers]
        self.v: List[torch.Tensor] = [torch.zeros(0, l.kv_heads, l.head_dim) for l in pkg.layers]
        self.conv: List[torch.Tensor] = []     # no recurrent layers: present so that the cold-copy code finds the fields
        self.ssm: List[torch.Tensor] = []
        self.n_tokens = 0


class PackageReference:
    def __init__(self, pkg: Package, weights: Dict[str, torch.Tensor], rms_eps: float = 1e-6):
        if any(l.kind not in (FULL, SLIDING) for l in pkg.layers):
            raise ValueError(f"{pkg.model_id}: this oracle runs attention-only schedules")
        self.pkg, self.eps = pkg, rms_eps
        self.w = {k: v.detach().float().cpu() for k, v in weights.items()}
        self.t = package_traits(pkg)

    def _attn(self, seq: PackageSequence, i: int, normed: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        l, w, t = self.pkg.layers[i], self.w, self.t
        p = f"text/layers/{i}"
        T, D = normed.shape[0], l.head_dim
        q = R.bf16_round(normed @ w[f"{p}/attn/q_proj"].t()).reshape(T, l.q_heads, D)
        k = R.bf16_round(normed @ w[f"{p}/attn/k_proj"].t()).reshape(T, l.kv_heads, D)
        shared_v = t["k_equals_v"] and l.kind == FULL
        v = k.clone() if shared_v else R.bf16_round(normed @ w[f"{p}/attn/v_proj"].t()).reshape(T, l.kv_heads, D)
        if t["qk_norm"]:
            q = R.bf16_round(R.rmsnorm(q, w[f"{p}/attn/q_norm"], self.eps, True))
            k = R.bf16_round(R.rmsnorm(k, w[f"{p}/attn/k_norm"], self.eps, True))
        if l.rotary_dim > 0:          # 0: a layer without positional rotation
            q = R.bf16_round(R.rope_partial(q, pos, l.rotary_dim, l.rope_theta))
            k = R.bf16_round(R.rope_partial(k, pos, l.rotary_dim, l.rope_theta))
        base = seq.k[i].shape[0]
        seq.k[i] = torch.cat([seq.k[i], k], 0)
        seq.v[i] = torch.cat([seq.v[i], v], 0)
        n = base + T
        vis = torch.arange(n)[None, :] <= (base + torch.arange(T))[:, None]              # causal
        if l.kind == SLIDING and l.window > 0:
            vis &= torch.arange(n)[None, :] > (base + torch.arange(T))[:, None] - l.window  # the last `window` keys
        o = R.gqa_attention(q, seq.k[i], seq.v[i], None, t["qk_scale"] / math.sqrt(D), vis)
        o = R.bf16_round(o)                                                              # [T, H, D]
        if t["headwise_gate"]:
            gate = torch.sigmoid(R.bf16_round(normed @ w[f"{p}/attn/gate"].t()))         # [T, H]: one gate per head
            o = R.bf16_round(o * gate[:, :, None])
        return R.bf16_round(o.reshape(T, l.q_heads * D) @ w[f"{p}/attn/o_proj"].t())

    def _mlp(self, i: int, normed: torch.Tensor) -> torch.Tensor:
        w, t = self.w, self.t
        p = f"text/layers/{i}"
        gu = normed @ w[f"{p}/mlp/gate_up"].t()
        half = gu.shape[1] // 2
        if t["geglu"]:
            act = torch.nn.functional.gelu(gu[:, :half], approximate="tanh" if t["gelu_tanh"] else "none")
        else:
            act = torch.nn.functional.silu(gu[:, :half])
        return R.bf16_round(act * gu[:, half:]) @ w[f"{p}/mlp/down"].t()

    def forward(self, seq: PackageSequence, ids: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        w, t = self.w, self.t
        T = ids.shape[0]
        pos = seq.n_tokens + torch.arange(T) if positions is None else positions
        x = w["text/embed"][ids.long()].float()
        for i in range(self.pkg.n_layers):
            p = f"text/layers/{i}"
            a = self._attn(seq, i, R.bf16_round(R.rmsnorm(x, w[f"{p}/input_norm"], self.eps, True)), pos)
            if t["post_branch_norms"]:
                a = R.bf16_round(R.rmsnorm(a, w[f"{p}/attn_out_norm"], self.eps, True))
            x = R.bf16_round(x + a)
            m = self._mlp(i, R.bf16_round(R.rmsnorm(x, w[f"{p}/post_norm"], self.eps, True)))
            if t["post_branch_norms"]:
                m = R.bf16_round(R.rmsnorm(m, w[f"{p}/mlp_out_norm"], self.eps, True))
            x = R.bf16_round(x + m)
        seq.n_tokens += T
        return R.bf16_round(R.rmsnorm(x, w["text/final_norm"], self.eps, True))

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        head = self.w["text/embed"] if self.pkg.tie_word_embeddings else self.w["text/lm_head"]
        lg = R.bf16_round(hidden.float() @ head.t()) * self.t["output_multiplier"]
        cap = self.pkg.final_logit_softcap
        return cap * torch.tanh(lg / cap) if cap > 0 else lg

    def generate_greedy(self, prompt: torch.Tensor, n_new: int) -> List[int]:
        seq = PackageSequence(self.pkg)
        h = self.forward(seq, prompt)
        out = [int(R.argmax_lowest(self.logits(h[-1:]))[0])]
        for _ in range(n_new - 1):
            h = self.forward(seq, torch.tensor([out[-1]]))
            out.append(int(R.argmax_lowest(self.logits(h))[0]))
        return out


def package_model_config(pkg: Package, max_context: int = 4096) -> ModelConfig:
    """A ModelConfig-shaped summary for code that only needs widths and limits (the Program base class)."""
    l0 = pkg.layers[0]
    return ModelConfig(name=pkg.model_id, n_layers=pkg.n_layers, hidden=pkg.hidden, vocab=pkg.vocab, n_q_heads=l0.q_heads,
                       n_kv_heads=l0.kv_heads, head_dim=l0.head_dim, rot_dim=l0.rotary_dim, rope_theta=l0.rope_theta or 1e4,
                       gdn_qk_heads=0, gdn_v_heads=0, ffn_inter=pkg.intermediate, full_attn_interval=1, mtp_layers=0,
                       max_context=max_context)
