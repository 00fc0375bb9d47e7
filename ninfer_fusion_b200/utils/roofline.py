"""Analytic decode roofline and tensor-parallel link model (host-only arithmetic).

`decode_roofline`: the reference's serving roofline, tok/s = bandwidth / (weight bytes + KV bytes(ctx) + recurrent
state bytes) per sequence-step (tools/roofline/serve_roofline.py:9-20), extended with the batch dimension and the
GDN state traffic of the hybrid decoder.  `tp_link_bytes`: payload bytes per decode step that cross the links for a
tensor- or expert-parallel plan (src/core/tp_link_model.h:198-262 is the reference's analytic counterpart).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

from ..models.config import ModelConfig

WEIGHT_BITS = {"bf16": 16.0, "fp8": 8.0 + 32.0 / 5120, "nvfp4": 4.5}
KV_BITS = {"bf16": 16.0, "fp8": 8.0 + 16.0 / 256, "int8": 8.0 + 16.0 / 64, "nvfp4": 4.5}


def measured_peaks(path: Optional[str] = None) -> Dict[str, float]:
    """Copy bandwidth (GB/s) and bf16 GEMM throughput (TFLOP/s) as measured on the target GPU (MEASURED_PEAKS.json beside the package), else a stated fallback."""
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def matmul_params(cfg: ModelConfig, include_head: bool = True) -> int:
    n = cfg.param_count() - cfg.vocab * cfg.hidden  # the embedding table is gathered, not streamed
    return n if include_head else n - cfg.vocab * cfg.hidden


def decode_roofline(cfg: ModelConfig, batch: int, ctx: int, weights: str = "bf16", kv: str = "fp8", world: int = 1,
                    hbm_gbs: Optional[float] = None) -> Dict[str, float]:
    """Bytes one GPU must move per decode round and the round time / tok/s that the copy bandwidth allows."""
    bw = (hbm_gbs or measured_peaks()["hbm_gbs"]) * 1e9
    if cfg.moe is None:
        w_bytes = matmul_params(cfg) * WEIGHT_BITS[weights] / 8 / world
    else:
        m = cfg.moe
        dense = matmul_params(cfg) - cfg.n_layers * m.n_experts * 3 * cfg.hidden * m.expert_inter
        touched = min(m.n_experts / world, batch * m.top_k)        # experts of this rank that see a token
        w_bytes = dense * WEIGHT_BITS[weights] / 8 + cfg.n_layers * touched * 3 * cfg.hidden * m.expert_inter * WEIGHT_BITS[weights] / 8
    b_local = batch if cfg.moe is None else batch / world          # EP runs attention data-parallel
    kv_heads = cfg.n_kv_heads / (world if cfg.moe is None else 1)
    kv_bytes = b_local * ctx * len(cfg.attn_layers) * 2 * max(kv_heads, 1) * cfg.head_dim * KV_BITS[kv] / 8
    v_heads = cfg.gdn_v_heads / (world if cfg.moe is None else 1)
    state_bytes = b_local * len(cfg.gdn_layers) * v_heads * cfg.gdn_head_dim ** 2 * 4 * 2   # read + write
    total = w_bytes + kv_bytes + state_bytes
    t = total / bw
    return {"weight_bytes": w_bytes, "kv_bytes": kv_bytes, "state_bytes": state_bytes, "round_ms": t * 1e3,
            "tok_s": batch / t}


def tp_link_bytes(cfg: ModelConfig, batch: int, world: int, plan: str = "tp") -> Dict[str, float]:
    """Payload bytes per decode round that one rank sends (fp32 partial tiles for the one-shot all-reduce, bf16
    rows for expert dispatch / return) and the time at the measured 770 GB/s per direction."""
    if world <= 1:
        return {"bytes_sent": 0.0, "link_ms": 0.0}
    if plan == "tp":
        # two row-parallel GEMMs per layer, each pushes its [batch, hidden] fp32 tile to every other rank
        sent = cfg.n_layers * 2 * batch * cfg.hidden * 4 * (world - 1)
    else:
        m = cfg.moe
        b_local = batch / world
        away = (world - 1) / world                                  # routes that leave the rank, uniform routing
        sent = cfg.n_layers * b_local * m.top_k * cfg.hidden * 2 * away * 2   # dispatch + the mirrored return
    return {"bytes_sent": float(sent), "link_ms": sent / 770e9 * 1e3}
