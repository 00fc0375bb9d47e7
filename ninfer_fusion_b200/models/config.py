"""Model geometry of the supported Qwen3.x hybrid decoders.

The closed set mirrors the reference's registered targets
(src/targets/qwen3_6_27b/impl/config.h:12-110, src/targets/qwen3_6_35b_a3b,
docs/maintainer/qwen3.6-27b-model.md:25-78, qwen3.6-35b-a3b-model.md:37-133):
a repeating pattern of 3 Gated-DeltaNet layers followed by 1 gated GQA layer,
dense SwiGLU or sparse-MoE feed-forward, a 1-layer MTP draft module.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional


@dataclass(frozen=True)
class MoEConfig:
    n_experts: int = 256
    top_k: int = 8
    expert_inter: int = 512
    shared_inter: int = 512  # one shared expert with a sigmoid scalar gate
    norm_topk: bool = True


@dataclass(frozen=True)
class ModelConfig:
    name: str
    n_layers: int
    hidden: int
    vocab: int
    # full-attention (GQA) layers
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    rot_dim: int  # rotary dims at the front of each head (partial NeoX)
    rope_theta: float
    # gated delta-net layers
    gdn_qk_heads: int
    gdn_v_heads: int
    gdn_head_dim: int = 128
    conv_kernel: int = 4
    # feed-forward
    ffn_inter: int = 0
    moe: Optional[MoEConfig] = None
    rms_eps: float = 1e-6
    full_attn_interval: int = 4  # layer i is full attention iff (i + 1) % interval == 0
    mrope_sections: tuple = (11, 11, 10)
    mtp_layers: int = 1
    max_context: int = 262144
    rope_yarn_factor: float = 0.0   # > 1: YaRN context extension by this factor over max_context (yarn4 = 4.0)

    # ---- derived geometry ----
    def is_full_attn(self, layer: int) -> bool:
        return (layer + 1) % self.full_attn_interval == 0

    @property
    def attn_layers(self) -> list[int]:
        return [i for i in range(self.n_layers) if self.is_full_attn(i)]

    @property
    def gdn_layers(self) -> list[int]:
        return [i for i in range(self.n_layers) if not self.is_full_attn(i)]

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def attn_in_dim(self) -> int:
        """Rows of the fused attention input projection: [query, key, output_gate, value]."""
        return 2 * self.q_dim + 2 * self.kv_dim

    @property
    def gdn_qk_dim(self) -> int:
        return self.gdn_qk_heads * self.gdn_head_dim

    @property
    def gdn_v_dim(self) -> int:
        return self.gdn_v_heads * self.gdn_head_dim

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_qk_dim + self.gdn_v_dim

    @property
    def gdn_in_dim(self) -> int:
        """Rows of the fused GDN input projection: [q, k, v, z, a, b]."""
        return self.gdn_conv_dim + self.gdn_v_dim + 2 * self.gdn_v_heads

    def param_count(self) -> int:
        h = self.hidden
        attn = self.attn_in_dim * h + h * self.q_dim
        gdn = self.gdn_in_dim * h + h * self.gdn_v_dim + self.gdn_conv_dim * self.conv_kernel
        if self.moe is None:
            ffn = 3 * h * self.ffn_inter
        else:
            m = self.moe
            ffn = m.n_experts * 3 * h * m.expert_inter + 3 * h * m.shared_inter + (m.n_experts + 1) * h
        n_attn = len(self.attn_layers)
        return n_attn * attn + (self.n_layers - n_attn) * gdn + self.n_layers * ffn + 2 * self.vocab * h

    def shrink(self, n_layers: int, **kw) -> "ModelConfig":
        return replace(self, name=f"{self.name}-{n_layers}L", n_layers=n_layers, **kw)


QWEN36_27B = ModelConfig(
    name="qwen3.6-27b", n_layers=64, hidden=5120, vocab=248320,
    n_q_heads=24, n_kv_heads=4, head_dim=256, rot_dim=64, rope_theta=1e7,
    gdn_qk_heads=16, gdn_v_heads=48, ffn_inter=17408,
)

QWEN36_35B_A3B = ModelConfig(
    name="qwen3.6-35b-a3b", n_layers=40, hidden=2048, vocab=248320,
    n_q_heads=16, n_kv_heads=2, head_dim=256, rot_dim=64, rope_theta=1e7,
    gdn_qk_heads=16, gdn_v_heads=32, ffn_inter=0, moe=MoEConfig(),
)

# The 3.5-generation 9B GDN hybrid (src/targets/qwen3_5_9b/impl/config.h:12-30: 32 layers, hidden 4096, 16 / 4 heads of
# 256, GDN 16 key / 32 value heads of 128, MLP 12288, one draft layer).
QWEN35_9B = ModelConfig(
    name="qwen3.5-9b", n_layers=32, hidden=4096, vocab=248320,
    n_q_heads=16, n_kv_heads=4, head_dim=256, rot_dim=64, rope_theta=1e7,
    gdn_qk_heads=16, gdn_v_heads=32, ffn_inter=12288,
)

# Small geometries with the same structure, for CPU oracles and GPU smoke runs.
TINY_DENSE = ModelConfig(
    name="tiny-dense", n_layers=4, hidden=256, vocab=1024,
    n_q_heads=6, n_kv_heads=1, head_dim=256, rot_dim=64, rope_theta=1e7,
    gdn_qk_heads=2, gdn_v_heads=6, ffn_inter=512, max_context=4096,
)

TINY_MOE = ModelConfig(
    name="tiny-moe", n_layers=4, hidden=256, vocab=1024,
    n_q_heads=8, n_kv_heads=1, head_dim=256, rot_dim=64, rope_theta=1e7,
    gdn_qk_heads=2, gdn_v_heads=4, ffn_inter=0,
    moe=MoEConfig(n_experts=16, top_k=4, expert_inter=128, shared_inter=128), max_context=4096,
)

REGISTRY = {c.name: c for c in (QWEN36_27B, QWEN36_35B_A3B, QWEN35_9B, TINY_DENSE, TINY_MOE)}
# The 3.8 generation shares the 27B geometry (docs/maintainer/qwen3.8-27b-artifact.md).
REGISTRY["qwen3.8-27b"] = replace(QWEN36_27B, name="qwen3.8-27b")


def get_config(name: str) -> ModelConfig:
    """Registered geometry by name; `name@N` is the same geometry shrunk to N layers (debug artifacts)."""
    if "@" in name:
        base, _, n = name.partition("@")
        return replace(get_config(base), n_layers=int(n), name=name)
    try:
        return REGISTRY[name]
    except KeyError:
        raise KeyError(f"unknown model '{name}'; registered: {sorted(REGISTRY)}") from None
