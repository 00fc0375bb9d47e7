"""GPU budget matrix: weight bytes per format, and the context each KV tier reaches in what is left."""
from __future__ import annotations

from typing import Dict, List

from ..models.config import ModelConfig

GPUS: Dict[str, Dict[str, float]] = {
    # memory in GiB usable by one process, copy bandwidth in TB/s (B200: a measured copy rate, not the nominal 7.7)
    "b200": {"mem_gib": 178.0, "tbps": 6.5},
    "h200": {"mem_gib": 139.0, "tbps": 4.0},
    "h100": {"mem_gib": 79.0, "tbps": 2.9},
    "rtx5090": {"mem_gib": 31.0, "tbps": 1.5},
}
WEIGHT_BITS = {"bf16": 16.0, "fp8": 8.0 + 16.0 / 5120, "nvfp4": 4.5, "q4": 4.25, "q5": 5.25, "q6": 6.25, "w8": 8.5}
KV_BITS = {"bf16": 16.0, "fp8": 8.0625, "int8": 8.25, "nvfp4": 4.5}   # per stored value, scales included


def budget_matrix(cfg: ModelConfig, world: int = 1, batch: int = 1, reserve_gib: float = 6.0) -> List[Dict]:
    """One row per (gpu, weight format): weight GiB per rank, whether it fits, decode roofline tok/s at batch 1, and
    the longest context (tokens per sequence at `batch` sequences) per KV tier in the remaining memory."""
    params = cfg.param_count()
    embed = 2 * cfg.vocab * cfg.hidden
    rows = []
    kv_values_per_token = 2 * len(cfg.attn_layers) * cfg.n_kv_heads * cfg.head_dim / world
    state_bytes = len(cfg.gdn_layers) * (cfg.gdn_v_heads * cfg.gdn_head_dim * cfg.gdn_head_dim * 4) / world
    for gpu, spec in GPUS.items():
        for fmt, bits in WEIGHT_BITS.items():
            wbytes = ((params - embed) * bits / 8 + embed * 2) / world      # embedding and head stay bf16
            left = spec["mem_gib"] * (1 << 30) - reserve_gib * (1 << 30) - wbytes - 2 * batch * state_bytes
            ctx = {tier: max(0, int(left / (batch * kv_values_per_token * b / 8))) if left > 0 else 0
                   for tier, b in KV_BITS.items()}
            rows.append({"gpu": gpu, "weights": fmt, "weight_gib": round(wbytes / (1 << 30), 2), "fits": left > 0,
                         "decode_tok_s_roofline": round(spec["tbps"] * 1e12 / wbytes, 1),
                         "max_context": ctx})
    return rows
