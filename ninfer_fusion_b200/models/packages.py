"""Closed table of model packages with a capability gate.

A package is a model id, its geometry, its per-layer schedule (full / sliding-window / NoPE attention, gated delta
net) and the list of runtime capabilities it needs.  ``construct`` refuses a package whose needs the engine does not
have and names the missing ones, instead of running a model with a layer kind silently skipped (the failure the
reference's scaffolded configs were rejected for).  The hybrid GDN family (`models/config.py`) is fully served; the
all-attention packages below are geometry-complete descriptions that the gate refuses until their layer kinds land.

Reference: src/targets/registry.{h,cpp} (closed model-id table, capability gate, construct_registered),
src/targets/declared_capabilities.h, src/targets/{spark_x2_5_4b,muse_glimmer_30b,gemma4_31b}/impl/config.h.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, FrozenSet, Optional, Tuple

from .config import REGISTRY, ModelConfig

FULL, SLIDING, GDN = "full", "sliding", "gdn"

# what the engine's forward pass, kernels and cache can do today
ENGINE_CAPABILITIES: FrozenSet[str] = frozenset({
    "gdn-hybrid-schedule",        # 3 GDN : 1 gated GQA layers
    "gated-attention-output",     # elementwise sigmoid gate on the attention output
    "qk-norm", "partial-rope", "mrope", "yarn",
    "swiglu-mlp", "sparse-moe", "mtp-draft",
    "sliding-window-attention",   # `window` in the prefill and split-KV decode kernels
    "head-dim-256", "head-dim-128",
    "kv:bf16", "kv:fp8", "kv:int8", "kv:nvfp4",
    "vision-tower",
})


@dataclass(frozen=True)
class LayerKind:
    kind: str                     # FULL | SLIDING | GDN
    rotary_dim: int = 0           # 0 = no positional rotation on this layer (NoPE)
    rope_theta: float = 0.0
    window: int = 0               # sliding layers
    q_heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0


@dataclass(frozen=True)
class Package:
    model_id: str
    hidden: int
    n_layers: int
    intermediate: int
    vocab: int
    layers: Tuple[LayerKind, ...]
    needs: FrozenSet[str]
    activation: str = "swiglu"
    final_logit_softcap: float = 0.0
    tie_word_embeddings: bool = False
    config: Optional[ModelConfig] = None      # set for packages the hybrid runtime serves
    notes: str = ""
    qk_scale: float = 1.0                     # learned-constant factor on q . k (on top of 1 / sqrt(head_dim))
    output_multiplier: float = 1.0            # factor on the logits before soft-capping

    def count(self, kind: str) -> int:
        return sum(1 for l in self.layers if l.kind == kind)

    def missing(self, have: FrozenSet[str] = ENGINE_CAPABILITIES) -> Tuple[str, ...]:
        return tuple(sorted(self.needs - have))


class PackageRefused(ValueError):
    pass


def _hybrid(cfg: ModelConfig) -> Package:
    kinds = tuple(LayerKind(FULL, cfg.rot_dim, cfg.rope_theta, 0, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim)
                  if cfg.is_full_attn(i) else LayerKind(GDN) for i in range(cfg.n_layers))
    needs = {"gdn-hybrid-schedule", "gated-attention-output", "qk-norm", "partial-rope", f"head-dim-{cfg.head_dim}",
             "sparse-moe" if cfg.moe is not None else "swiglu-mlp"}
    if cfg.mtp_layers:
        needs.add("mtp-draft")
    inter = cfg.ffn_inter if cfg.moe is None else cfg.moe.expert_inter
    return Package(cfg.name, cfg.hidden, cfg.n_layers, inter, cfg.vocab, kinds, frozenset(needs), config=cfg)


def _spark() -> Package:
    # 36 layers: every fourth is full attention (64 rotary dims, theta 5e6), the rest slide over 512 tokens with all
    # 256 dims rotated at theta 1e4; one attention geometry (16 / 4 heads of 256) for all layers
    kinds = tuple(LayerKind(FULL, 64, 5e6, 0, 16, 4, 256) if (i + 1) % 4 == 0 else LayerKind(SLIDING, 256, 1e4, 512, 16, 4, 256)
                  for i in range(36))
    return Package("spark-x2.5-4b", 2560, 36, 10240, 131072, kinds,
                   frozenset({"sliding-window-attention", "head-dim-256", "per-layer-rope", "headwise-attention-gate",
                              "geglu-mlp", "all-attention-schedule"}),
                   activation="gelu", tie_word_embeddings=True,
                   notes="no q/k norm, head-wise output gate (one gate row per query head), no draft layers")


def _muse() -> Package:
    # 52 layers: three sliding layers (window 2048, theta 5e5, all 128 dims rotated) then one full layer without any
    # positional rotation; logits soft-capped at 20, q.k scaled by a learned-constant factor, post-norms on both branches
    kinds = tuple(LayerKind(FULL, 0, 0.0, 0, 32, 2, 128) if (i + 1) % 4 == 0 else LayerKind(SLIDING, 128, 5e5, 2048, 32, 2, 128)
                  for i in range(52))
    return Package("muse-glimmer-30b", 6656, 52, 19968, 202048, kinds,
                   frozenset({"sliding-window-attention", "head-dim-128", "nope-layers", "logit-softcap", "qk-norm",
                              "post-branch-norms", "qk-scale-factor", "all-attention-schedule", "swiglu-mlp"}),
                   final_logit_softcap=20.0, output_multiplier=0.19611613513818404,
                   notes="output multiplier 0.19611613513818404, vocab rows padded to 202112")


def _gemma() -> Package:
    # 60 layers, two attention geometries: sliding (32 / 16 heads of 256, window 1024, theta 1e4) and every sixth layer
    # full (32 / 4 heads of 512, 128 rotary dims, theta 1e6, K shared with V)
    kinds = tuple(LayerKind(FULL, 128, 1e6, 0, 32, 4, 512) if (i + 1) % 6 == 0 else LayerKind(SLIDING, 256, 1e4, 1024, 32, 16, 256)
                  for i in range(60))
    return Package("gemma4-31b", 5376, 60, 21504, 262144, kinds,
                   frozenset({"sliding-window-attention", "head-dim-256", "head-dim-512", "per-layer-attention-geometry",
                              "per-layer-rope", "logit-softcap", "k-equals-v", "geglu-mlp", "all-attention-schedule"}),
                   activation="gelu_pytorch_tanh", final_logit_softcap=30.0, tie_word_embeddings=True,
                   notes="skeleton in the reference as well: two head widths cannot be one flat attention geometry")


def _table() -> Dict[str, Package]:
    out = {name: _hybrid(cfg) for name, cfg in REGISTRY.items()}
    for p in (_spark(), _muse(), _gemma()):
        out[p.model_id] = p
    return out


PACKAGES: Dict[str, Package] = _table()


def lookup(model_id: str) -> Package:
    if model_id not in PACKAGES:
        raise PackageRefused(f"unknown model id '{model_id}' (registered: {', '.join(sorted(PACKAGES))})")
    return PACKAGES[model_id]


def construct(model_id: str, have: FrozenSet[str] = ENGINE_CAPABILITIES) -> ModelConfig:
    """The startup gate: the runtime config of a registered package, or a refusal that names what is missing."""
    p = lookup(model_id)
    miss = p.missing(have)
    if miss:
        raise PackageRefused(f"{model_id}: the engine lacks {', '.join(miss)}")
    if p.config is None:
        raise PackageRefused(f"{model_id}: registered as a geometry description only")
    if sum(p.count(k) for k in (FULL, SLIDING, GDN)) != p.n_layers:
        raise PackageRefused(f"{model_id}: the layer table does not cover all {p.n_layers} layers")
    return p.config


def construct_oracle(model_id: str, layers: int = 0, vocab: int = 0, hidden_div: int = 1) -> Package:
    """The package as the CPU oracle runtime serves it (models/all_attention.py): attention-only schedules, whatever
    the GPU gate says about them.  `model_id@N` or `layers` takes the first N layers of the schedule."""
    base, _, n = model_id.partition("@")
    p = lookup(base)
    if p.count(GDN):
        raise PackageRefused(f"{base}: a GDN hybrid is served by the hybrid runtime, not by the attention-only oracle")
    n_layers = int(n) if n else int(layers)
    if n_layers or vocab or hidden_div > 1:
        from .all_attention import shrink_package
        p = shrink_package(p, n_layers or p.n_layers, vocab or None, hidden_div)
    return p


def describe(model_id: str) -> dict:
    p = lookup(model_id)
    return {"model_id": p.model_id, "hidden": p.hidden, "layers": p.n_layers, "full": p.count(FULL),
            "sliding": p.count(SLIDING), "gdn": p.count(GDN), "intermediate": p.intermediate, "vocab": p.vocab,
            "activation": p.activation, "final_logit_softcap": p.final_logit_softcap,
            "needs": sorted(p.needs), "missing": list(p.missing()), "servable": not p.missing() and p.config is not None,
            "oracle_runtime": p.count(GDN) == 0 or p.config is not None, "notes": p.notes}
