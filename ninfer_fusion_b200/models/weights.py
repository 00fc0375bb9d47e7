"""Weight inventory of a hybrid decoder and random initialisation.

Tensor names and fused row orders follow the reference's artifact inventory
(docs/maintainer/qwen3.8-27b-artifact.md:71-127,194-284): the attention input
projection is one parent with rows ``[query, key, output_gate, value]``, the GDN
input projection ``[q, k, v, z]`` followed by the ``[A, B]`` gating rows, the MLP
parent ``[gate, up]``.  Fusing the tiny A/B projection into the GDN parent is a
load-time concatenation (the container keeps them as separate objects).
"""
from __future__ import annotations

from typing import Dict, Iterator, Tuple

import torch

from .config import ModelConfig


def weight_shapes(cfg: ModelConfig, with_mtp: bool = False) -> Iterator[Tuple[str, tuple, torch.dtype]]:
    h = cfg.hidden
    yield "text/embed", (cfg.vocab, h), torch.bfloat16
    yield "text/lm_head", (cfg.vocab, h), torch.bfloat16
    yield "text/final_norm", (h,), torch.bfloat16
    layer_sets = [("text/layers", cfg.n_layers, None)]
    if with_mtp:
        layer_sets.append(("mtp/layers", cfg.mtp_layers, "attn"))
        yield "mtp/fc", (h, 2 * h), torch.bfloat16          # [hidden ; embedding] -> hidden
        yield "mtp/pre_fc_norm_hidden", (h,), torch.bfloat16
        yield "mtp/pre_fc_norm_embedding", (h,), torch.bfloat16
        yield "mtp/final_norm", (h,), torch.bfloat16
    for prefix, n, force in layer_sets:
        for i in range(n):
            p = f"{prefix}/{i}"
            yield f"{p}/input_norm", (h,), torch.bfloat16
            yield f"{p}/post_norm", (h,), torch.bfloat16
            if force == "attn" or (force is None and cfg.is_full_attn(i)):
                yield f"{p}/attn/in_proj", (cfg.attn_in_dim, h), torch.bfloat16
                yield f"{p}/attn/q_norm", (cfg.head_dim,), torch.bfloat16
                yield f"{p}/attn/k_norm", (cfg.head_dim,), torch.bfloat16
                yield f"{p}/attn/o_proj", (h, cfg.q_dim), torch.bfloat16
            else:
                yield f"{p}/gdn/in_proj", (cfg.gdn_in_dim, h), torch.bfloat16
                yield f"{p}/gdn/conv_w", (cfg.gdn_conv_dim, cfg.conv_kernel), torch.bfloat16
                yield f"{p}/gdn/A_log", (cfg.gdn_v_heads,), torch.float32
                yield f"{p}/gdn/dt_bias", (cfg.gdn_v_heads,), torch.float32
                yield f"{p}/gdn/norm", (cfg.gdn_head_dim,), torch.bfloat16
                yield f"{p}/gdn/out_proj", (h, cfg.gdn_v_dim), torch.bfloat16
            if cfg.moe is None:
                yield f"{p}/mlp/gate_up", (2 * cfg.ffn_inter, h), torch.bfloat16
                yield f"{p}/mlp/down", (h, cfg.ffn_inter), torch.bfloat16
            else:
                m = cfg.moe
                yield f"{p}/moe/router", (m.n_experts + 1, h), torch.bfloat16  # last row: shared-expert gate
                yield f"{p}/moe/experts_gate_up", (m.n_experts, 2 * m.expert_inter, h), torch.bfloat16
                yield f"{p}/moe/experts_down", (m.n_experts, h, m.expert_inter), torch.bfloat16
                yield f"{p}/moe/shared_gate_up", (2 * m.shared_inter, h), torch.bfloat16
                yield f"{p}/moe/shared_down", (h, m.shared_inter), torch.bfloat16


def random_weights(cfg: ModelConfig, device, seed: int = 0, with_mtp: bool = False,
                   std: float = 0.02, expert_rank: int = 0, expert_world: int = 1,
                   weight_format: str = "bf16") -> Dict[str, torch.Tensor]:
    """Random-init weights of the architecture (there are no checkpoints on the box).

    With `expert_world` > 1 the routed expert banks hold only this rank's contiguous range of experts
    (drawn from a rank-specific stream); every other tensor is identical on all ranks.
    """
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    gen_experts = torch.Generator(device=device)
    gen_experts.manual_seed(seed * 1000 + 31 + expert_rank)
    out: Dict[str, torch.Tensor] = {}
    for name, shape, dt in weight_shapes(cfg, with_mtp):
        if expert_world > 1 and name.rsplit("/", 1)[-1] in ("experts_gate_up", "experts_down"):
            t = torch.empty((shape[0] // expert_world,) + tuple(shape[1:]), dtype=dt, device=device)
            t.normal_(0.0, std, generator=gen_experts)
            out[name] = t
            continue
        t = torch.empty(shape, dtype=dt, device=device)
        leaf = name.rsplit("/", 1)[-1]
        if leaf.endswith("norm") or leaf in ("q_norm", "k_norm", "pre_fc_norm_hidden", "pre_fc_norm_embedding"):
            # unit-offset norms store w - 1; the GDN head norm stores w
            t.normal_(0.0, 0.02, generator=gen)
            if name.endswith("gdn/norm"):
                t.add_(1.0)
        elif leaf == "A_log":
            t.uniform_(-1.0, 1.5, generator=gen)
        elif leaf == "dt_bias":
            t.uniform_(-2.0, 1.0, generator=gen)
        elif leaf == "conv_w":
            t.normal_(0.0, 0.3, generator=gen)
        else:
            t.normal_(0.0, std, generator=gen)
        out[name] = quantize_tensor(name, t, weight_format)  # quantised right away: the bf16 copy is dropped
    return out


QUANT_LEAVES = ("in_proj", "o_proj", "out_proj", "gate_up", "down", "lm_head")
GROUPINT_FORMATS = ("q4", "q5", "q6", "w8")   # groupwise-int codes kept as the artifact stores them (ops.groupint)


def quantize_tensor(name: str, t: torch.Tensor, weight_format: str):
    """bf16 matmul weight -> QuantWeight for the tcgen05 quantised GEMMs ('fp8' row-scale or 'nvfp4' block-scaled).
    The fused [gate; up] parent is stored tile-interleaved, as the quantised SwiGLU epilogue expects."""
    from ..ops import quant as Q
    from .hybrid import QuantWeight
    leaf = name.rsplit("/", 1)[-1]
    if weight_format == "bf16" or t.dim() != 2 or leaf not in QUANT_LEAVES or "/moe/" in name:
        return t
    N, K = t.shape
    fmt, _, rot = weight_format.partition("+h")       # "q4+h64": Q4 codes of the weight with its input rotated
    if fmt in GROUPINT_FORMATS:
        from ..ops.groupint import GroupIntWeight
        rot_block = int(rot) if rot else 0
        if rot_block and K % rot_block:
            rot_block = 0                                 # widths the block does not divide stay unrotated
        return GroupIntWeight.from_dense(t, fmt, rot_block=rot_block)
    w = Q.interleave_gate_up(t) if leaf == "gate_up" else t
    if weight_format == "fp8":
        codes, scale = Q.quantize_fp8_row(w)
        return QuantWeight(Q.QT_FP8_ROW, codes, scale, 1.0, (N, K))
    if weight_format == "nvfp4":
        if K % 256:
            # zero columns up to the kernel's 256-value k-block (sharded down projections); the consumer reads a
            # zero-padded activation of the same width
            Kp = (K + 255) // 256 * 256
            w = torch.cat([w, torch.zeros((N, Kp - K), dtype=w.dtype, device=w.device)], dim=1)
            K = Kp
        codes, plane, d_w = Q.quantize_nvfp4_prepare(w)
        return QuantWeight(Q.QT_NVFP4, codes, plane, d_w, (N, K))
    raise ValueError(f"unknown weight format '{weight_format}'")


def quantize_weights(weights: Dict[str, torch.Tensor], weight_format: str) -> Dict[str, object]:
    """Quantise every eligible matmul weight in place of its bf16 tensor (embedding, norms, conv, router stay bf16)."""
    return {k: quantize_tensor(k, v, weight_format) for k, v in weights.items()}


def dequantize_weights(weights: Dict[str, object]) -> Dict[str, torch.Tensor]:
    """The represented values of every tensor (fp32 for quantised ones, original row order): the oracle's weights."""
    from ..ops import quant as Q
    out = {}
    for name, t in weights.items():
        if not hasattr(t, "qtype"):
            out[name] = t
            continue
        N, K = t.shape
        if t.qtype == 3:   # ops.groupint.GroupIntWeight
            out[name] = t.dequant().to(t.payload.device)
            continue
        w = Q.dequant_nvfp4(t.codes, t.scale, t.divisor, N, K) if t.qtype == Q.QT_NVFP4 else Q.dequant_fp8_row(t.codes, t.scale)
        out[name] = Q.deinterleave_gate_up(w) if name.endswith("gate_up") else w
    return out


def total_bytes(weights: Dict[str, object]) -> int:
    return sum(t.nbytes() if hasattr(t, "qtype") else t.numel() * t.element_size() for t in weights.values())
