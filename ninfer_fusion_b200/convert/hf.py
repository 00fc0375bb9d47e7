"""Hugging Face checkpoint <-> engine weight inventory for the hybrid GDN / gated-attention family.

Source names and transforms (tools/convert/qwen3_6_27b/recipe.py:55-235, tools/convert/qwen3_6_35b_a3b/recipe.py:50-105,
tools/convert/qwen3_6/common/recipe.py:110-125,200-265):

* `self_attn.q_proj.weight` is head-interleaved [heads, (query 256 | gate 256), hidden]; the engine's fused input
  projection is [query, key, output_gate, value];
* the GDN parent is [in_proj_qkv (q, k, v) ; in_proj_z ; in_proj_a ; in_proj_b]; `conv1d.weight` [C, 1, 4] drops
  its middle axis; `A_log` / `dt_bias` become fp32;
* the MLP parent is [gate_proj ; up_proj]; MoE: router = [gate.weight ; shared_expert_gate.weight], routed banks
  are already expert-major with [gate ; up] halves;
* the draft module: `mtp.fc`, `mtp.pre_fc_norm_{hidden,embedding}`, `mtp.norm`, `mtp.layers.0.*`;
* the vision tower: `model.visual.*` (patch projection flattened to [1152, 1536]).

`weights_to_hf` is the exact inverse (export, and the round-trip test of this mapping).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterator, Optional, Tuple

import torch

from ..models.config import ModelConfig
from ..models.vision import VisionConfig

TEXT = "model.language_model."
VISUAL = "model.visual."


def _split_q_gate(q_proj: torch.Tensor, heads: int, D: int) -> Tuple[torch.Tensor, torch.Tensor]:
    per_head = q_proj.view(heads, 2 * D, -1)
    return per_head[:, :D].reshape(heads * D, -1), per_head[:, D:].reshape(heads * D, -1)


def _join_q_gate(q: torch.Tensor, gate: torch.Tensor, heads: int, D: int) -> torch.Tensor:
    return torch.cat([q.view(heads, D, -1), gate.view(heads, D, -1)], dim=1).reshape(2 * heads * D, -1)


def _layer_leaves(cfg: ModelConfig, get: Callable[[str], torch.Tensor], src: str, dst: str, attn: bool
                  ) -> Iterator[Tuple[str, torch.Tensor]]:
    bf = torch.bfloat16
    yield f"{dst}/input_norm", get(src + "input_layernorm.weight").to(bf)
    yield f"{dst}/post_norm", get(src + "post_attention_layernorm.weight").to(bf)
    if attn:
        q, gate = _split_q_gate(get(src + "self_attn.q_proj.weight"), cfg.n_q_heads, cfg.head_dim)
        yield f"{dst}/attn/in_proj", torch.cat([q, get(src + "self_attn.k_proj.weight"), gate,
                                                get(src + "self_attn.v_proj.weight")]).to(bf).contiguous()
        yield f"{dst}/attn/q_norm", get(src + "self_attn.q_norm.weight").to(bf)
        yield f"{dst}/attn/k_norm", get(src + "self_attn.k_norm.weight").to(bf)
        yield f"{dst}/attn/o_proj", get(src + "self_attn.o_proj.weight").to(bf)
    else:
        la = src + "linear_attn."
        yield f"{dst}/gdn/in_proj", torch.cat([get(la + "in_proj_qkv.weight"), get(la + "in_proj_z.weight"),
                                               get(la + "in_proj_a.weight"), get(la + "in_proj_b.weight")]).to(bf).contiguous()
        yield f"{dst}/gdn/conv_w", get(la + "conv1d.weight")[:, 0, :].to(bf).contiguous()
        yield f"{dst}/gdn/A_log", get(la + "A_log").float()
        yield f"{dst}/gdn/dt_bias", get(la + "dt_bias").float()
        yield f"{dst}/gdn/norm", get(la + "norm.weight").to(bf)
        yield f"{dst}/gdn/out_proj", get(la + "out_proj.weight").to(bf)
    m = src + "mlp."
    if cfg.moe is None:
        yield f"{dst}/mlp/gate_up", torch.cat([get(m + "gate_proj.weight"), get(m + "up_proj.weight")]).to(bf).contiguous()
        yield f"{dst}/mlp/down", get(m + "down_proj.weight").to(bf)
    else:
        yield f"{dst}/moe/router", torch.cat([get(m + "gate.weight"), get(m + "shared_expert_gate.weight")]).to(bf).contiguous()
        yield f"{dst}/moe/experts_gate_up", get(m + "experts.gate_up_proj").to(bf)
        yield f"{dst}/moe/experts_down", get(m + "experts.down_proj").to(bf)
        yield f"{dst}/moe/shared_gate_up", torch.cat([get(m + "shared_expert.gate_proj.weight"),
                                                     get(m + "shared_expert.up_proj.weight")]).to(bf).contiguous()
        yield f"{dst}/moe/shared_down", get(m + "shared_expert.down_proj.weight").to(bf)


def hf_to_weights(cfg: ModelConfig, source, with_mtp: bool = False, vision: Optional[VisionConfig] = None
                  ) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (engine leaf name, tensor) one leaf at a time.  `source` has `.tensor(name)` and `in`."""
    get = source.tensor
    bf = torch.bfloat16
    yield "text/embed", get(TEXT + "embed_tokens.weight").to(bf)
    head = "lm_head.weight" if "lm_head.weight" in source else TEXT + "embed_tokens.weight"   # tied embeddings
    yield "text/lm_head", get(head).to(bf)
    yield "text/final_norm", get(TEXT + "norm.weight").to(bf)
    for i in range(cfg.n_layers):
        yield from _layer_leaves(cfg, get, f"{TEXT}layers.{i}.", f"text/layers/{i}", cfg.is_full_attn(i))
    if with_mtp:
        yield "mtp/fc", get("mtp.fc.weight").to(bf)
        yield "mtp/pre_fc_norm_hidden", get("mtp.pre_fc_norm_hidden.weight").to(bf)
        yield "mtp/pre_fc_norm_embedding", get("mtp.pre_fc_norm_embedding.weight").to(bf)
        yield "mtp/final_norm", get("mtp.norm.weight").to(bf)
        for i in range(cfg.mtp_layers):
            yield from _layer_leaves(cfg, get, f"mtp.layers.{i}.", f"mtp/layers/{i}", True)
    if vision is not None:
        v = VISUAL
        yield "vision/patch_embed", get(v + "patch_embed.proj.weight").reshape(vision.hidden, vision.patch_dim).to(bf).contiguous()
        yield "vision/patch_embed_bias", get(v + "patch_embed.proj.bias").to(bf)
        yield "vision/pos_embed", get(v + "pos_embed.weight").to(bf)
        for l in range(vision.layers):
            s, d = f"{v}blocks.{l}.", f"vision/blocks/{l}"
            for ours, theirs in (("norm1_w", "norm1.weight"), ("norm1_b", "norm1.bias"), ("qkv", "attn.qkv.weight"),
                                 ("qkv_bias", "attn.qkv.bias"), ("proj", "attn.proj.weight"), ("proj_bias", "attn.proj.bias"),
                                 ("norm2_w", "norm2.weight"), ("norm2_b", "norm2.bias"), ("fc1", "mlp.linear_fc1.weight"),
                                 ("fc1_bias", "mlp.linear_fc1.bias"), ("fc2", "mlp.linear_fc2.weight"),
                                 ("fc2_bias", "mlp.linear_fc2.bias")):
                yield f"{d}/{ours}", get(s + theirs).to(bf)
        for ours, theirs in (("norm_w", "norm.weight"), ("norm_b", "norm.bias"), ("fc1", "linear_fc1.weight"),
                             ("fc1_bias", "linear_fc1.bias"), ("fc2", "linear_fc2.weight"), ("fc2_bias", "linear_fc2.bias")):
            yield f"vision/merger/{ours}", get(v + "merger." + theirs).to(bf)


def _layer_to_hf(cfg: ModelConfig, w: Dict[str, torch.Tensor], src: str, dst: str, attn: bool, out: Dict[str, torch.Tensor]) -> None:
    out[dst + "input_layernorm.weight"] = w[f"{src}/input_norm"]
    out[dst + "post_attention_layernorm.weight"] = w[f"{src}/post_norm"]
    if attn:
        p = w[f"{src}/attn/in_proj"]
        qd, kd = cfg.q_dim, cfg.kv_dim
        q, k, gate, v = p[:qd], p[qd:qd + kd], p[qd + kd:2 * qd + kd], p[2 * qd + kd:]
        out[dst + "self_attn.q_proj.weight"] = _join_q_gate(q, gate, cfg.n_q_heads, cfg.head_dim)
        out[dst + "self_attn.k_proj.weight"] = k
        out[dst + "self_attn.v_proj.weight"] = v
        out[dst + "self_attn.q_norm.weight"] = w[f"{src}/attn/q_norm"]
        out[dst + "self_attn.k_norm.weight"] = w[f"{src}/attn/k_norm"]
        out[dst + "self_attn.o_proj.weight"] = w[f"{src}/attn/o_proj"]
    else:
        p, la = w[f"{src}/gdn/in_proj"], dst + "linear_attn."
        C, vd, hv = cfg.gdn_conv_dim, cfg.gdn_v_dim, cfg.gdn_v_heads
        out[la + "in_proj_qkv.weight"] = p[:C]
        out[la + "in_proj_z.weight"] = p[C:C + vd]
        out[la + "in_proj_a.weight"] = p[C + vd:C + vd + hv]
        out[la + "in_proj_b.weight"] = p[C + vd + hv:]
        out[la + "conv1d.weight"] = w[f"{src}/gdn/conv_w"][:, None, :]
        out[la + "A_log"] = w[f"{src}/gdn/A_log"]
        out[la + "dt_bias"] = w[f"{src}/gdn/dt_bias"]
        out[la + "norm.weight"] = w[f"{src}/gdn/norm"]
        out[la + "out_proj.weight"] = w[f"{src}/gdn/out_proj"]
    m = dst + "mlp."
    if cfg.moe is None:
        gu = w[f"{src}/mlp/gate_up"]
        out[m + "gate_proj.weight"], out[m + "up_proj.weight"] = gu[:cfg.ffn_inter], gu[cfg.ffn_inter:]
        out[m + "down_proj.weight"] = w[f"{src}/mlp/down"]
    else:
        r, E = w[f"{src}/moe/router"], cfg.moe.n_experts
        out[m + "gate.weight"], out[m + "shared_expert_gate.weight"] = r[:E], r[E:]
        out[m + "experts.gate_up_proj"] = w[f"{src}/moe/experts_gate_up"]
        out[m + "experts.down_proj"] = w[f"{src}/moe/experts_down"]
        sgu = w[f"{src}/moe/shared_gate_up"]
        out[m + "shared_expert.gate_proj.weight"] = sgu[:cfg.moe.shared_inter]
        out[m + "shared_expert.up_proj.weight"] = sgu[cfg.moe.shared_inter:]
        out[m + "shared_expert.down_proj.weight"] = w[f"{src}/moe/shared_down"]


def weights_to_hf(cfg: ModelConfig, w: Dict[str, torch.Tensor], vision: Optional[VisionConfig] = None) -> Dict[str, torch.Tensor]:
    """Engine inventory (bf16 tensors) -> Hugging Face names and layouts."""
    out: Dict[str, torch.Tensor] = {TEXT + "embed_tokens.weight": w["text/embed"], "lm_head.weight": w["text/lm_head"],
                                    TEXT + "norm.weight": w["text/final_norm"]}
    for i in range(cfg.n_layers):
        _layer_to_hf(cfg, w, f"text/layers/{i}", f"{TEXT}layers.{i}.", cfg.is_full_attn(i), out)
    if "mtp/fc" in w:
        out["mtp.fc.weight"] = w["mtp/fc"]
        out["mtp.pre_fc_norm_hidden.weight"] = w["mtp/pre_fc_norm_hidden"]
        out["mtp.pre_fc_norm_embedding.weight"] = w["mtp/pre_fc_norm_embedding"]
        out["mtp.norm.weight"] = w["mtp/final_norm"]
        for i in range(cfg.mtp_layers):
            _layer_to_hf(cfg, w, f"mtp/layers/{i}", f"mtp.layers.{i}.", True, out)
    if vision is not None:
        v = VISUAL
        out[v + "patch_embed.proj.weight"] = w["vision/patch_embed"].view(vision.hidden, vision.channels, vision.temporal,
                                                                          vision.patch, vision.patch)
        out[v + "patch_embed.proj.bias"] = w["vision/patch_embed_bias"]
        out[v + "pos_embed.weight"] = w["vision/pos_embed"]
        for l in range(vision.layers):
            s, d = f"vision/blocks/{l}", f"{v}blocks.{l}."
            for ours, theirs in (("norm1_w", "norm1.weight"), ("norm1_b", "norm1.bias"), ("qkv", "attn.qkv.weight"),
                                 ("qkv_bias", "attn.qkv.bias"), ("proj", "attn.proj.weight"), ("proj_bias", "attn.proj.bias"),
                                 ("norm2_w", "norm2.weight"), ("norm2_b", "norm2.bias"), ("fc1", "mlp.linear_fc1.weight"),
                                 ("fc1_bias", "mlp.linear_fc1.bias"), ("fc2", "mlp.linear_fc2.weight"),
                                 ("fc2_bias", "mlp.linear_fc2.bias")):
                out[d + theirs] = w[f"{s}/{ours}"]
        for ours, theirs in (("norm_w", "norm.weight"), ("norm_b", "norm.bias"), ("fc1", "linear_fc1.weight"),
                             ("fc1_bias", "linear_fc1.bias"), ("fc2", "linear_fc2.weight"), ("fc2_bias", "linear_fc2.bias")):
            out[v + "merger." + theirs] = w[f"vision/merger/{ours}"]
    return {k: t.contiguous() for k, t in out.items()}


def config_from_hf(cfg_json: dict, name: str = "hf-import") -> ModelConfig:
    """ModelConfig from a Hugging Face config.json of this family (text_config of a VL wrapper, or flat)."""
    from ..models.config import MoEConfig
    t = cfg_json.get("text_config", cfg_json)
    rope = t.get("rope_parameters") or t.get("rope_scaling") or {}
    head_dim = int(t.get("head_dim", 256))
    rot = int(round(head_dim * float(t.get("partial_rotary_factor", rope.get("partial_rotary_factor", 0.25)))))
    moe = None
    if int(t.get("num_experts", 0)) > 0:
        moe = MoEConfig(n_experts=int(t["num_experts"]), top_k=int(t["num_experts_per_tok"]),
                        expert_inter=int(t["moe_intermediate_size"]), shared_inter=int(t["shared_expert_intermediate_size"]))
    return ModelConfig(
        name=name, n_layers=int(t["num_hidden_layers"]), hidden=int(t["hidden_size"]), vocab=int(t["vocab_size"]),
        n_q_heads=int(t["num_attention_heads"]), n_kv_heads=int(t["num_key_value_heads"]), head_dim=head_dim, rot_dim=rot,
        rope_theta=float(t.get("rope_theta", rope.get("rope_theta", 1e7))),
        gdn_qk_heads=int(t.get("linear_num_key_heads", 16)), gdn_v_heads=int(t.get("linear_num_value_heads", 32)),
        ffn_inter=0 if moe else int(t["intermediate_size"]), moe=moe)
