"""Model import assistant: what is this path, can this engine serve it, what fits on which GPU, and how to start it.

Recognises a Hugging Face checkpoint directory (`config.json` + `*.safetensors`), a GGUF file, or a `.ninfer` artifact;
maps it to a registered geometry or describes it through `adapt_config`; asks the capability gate and the geometry
gates; sizes weights and KV for a target GPU and context with the same arithmetic as the budget matrix; and prints the
command lines that follow (convert, then serve).  It reads headers and JSON only: no weights are loaded, no GPU is
opened.

Reference: tools/gui/model_import.py (recognise / judge / VRAM fit behind the GUI's "paste a model path" page),
tools/gui/gpu_compat.py, tools/gui/kv_tiers.py.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional

from ..models.config import REGISTRY, ModelConfig
from .adapt import AdaptError, adapt_config
from .gates import geometry_gates
from .matrix import GPUS, KV_BITS, WEIGHT_BITS


def recognise(path: str) -> Dict:
    """{"kind": "hf" | "gguf" | "ninfer" | "unknown", ...} from names and headers only."""
    if os.path.isdir(path):
        cfg = os.path.join(path, "config.json")
        shards = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        if os.path.exists(cfg):
            with open(cfg, encoding="utf-8") as f:
                hf = json.load(f)
            return {"kind": "hf", "config": hf, "shards": len(shards),
                    "bytes": sum(os.path.getsize(os.path.join(path, s)) for s in shards),
                    "has_tokenizer": os.path.exists(os.path.join(path, "tokenizer.json"))}
        return {"kind": "unknown", "why": "a directory without config.json"}
    if not os.path.isfile(path):
        return {"kind": "unknown", "why": "no such file or directory"}
    with open(path, "rb") as f:
        head = f.read(16)
    if head[:4] == b"GGUF":
        version, = struct.unpack_from("<I", head, 4)
        return {"kind": "gguf", "version": int(version), "bytes": os.path.getsize(path)}
    if path.endswith(".ninfer"):
        from ..artifact.container import ArtifactReader
        try:
            with ArtifactReader(path) as rd:
                return {"kind": "ninfer", "model_id": rd.identity[0], "weights_id": rd.identity[1],
                        "bytes": os.path.getsize(path)}
        except Exception as e:  # noqa: BLE001 - any malformed container is "unknown" with its reason
            return {"kind": "unknown", "why": f"not a readable artifact: {e}"}
    return {"kind": "unknown", "why": "neither a checkpoint directory, a GGUF file nor a .ninfer artifact"}


def match_registered(desc: Dict) -> Optional[ModelConfig]:
    """The registered geometry with the same layer count, width, head geometry and feed-forward shape, if any."""
    for cfg in REGISTRY.values():
        if cfg.name.startswith("tiny"):
            continue
        if (cfg.n_layers, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim) == (
                desc.get("layers"), desc.get("hidden"), desc.get("q_heads"), desc.get("kv_heads"), desc.get("head_dim")):
            return cfg
    return None


def fit(cfg: ModelConfig, gpu: str = "b200", context: int = 32768, lanes: int = 8, world: int = 1,
        reserve_gib: float = 6.0) -> List[Dict]:
    """One row per weight format: weight GiB per rank, the KV tiers whose pool for `lanes` x `context` tokens fits in
    what is left, and the widest tier that does."""
    spec = GPUS[gpu]
    params, embed = cfg.param_count(), 2 * cfg.vocab * cfg.hidden
    kv_values = 2 * len(cfg.attn_layers) * cfg.n_kv_heads * cfg.head_dim / world
    state = len(cfg.gdn_layers) * (cfg.gdn_v_heads * cfg.gdn_head_dim * cfg.gdn_head_dim * 4) / world
    rows = []
    for fmt, bits in WEIGHT_BITS.items():
        wbytes = ((params - embed) * bits / 8 + embed * 2) / world
        left = (spec["mem_gib"] - reserve_gib) * (1 << 30) - wbytes - 2 * lanes * state
        tiers = [t for t, b in sorted(KV_BITS.items(), key=lambda kv: -kv[1]) if left > 0 and lanes * context * kv_values * b / 8 <= left]
        rows.append({"weights": fmt, "weight_gib": round(wbytes / (1 << 30), 2), "fits": bool(tiers),
                     "kv_tiers_that_fit": tiers, "widest_kv": tiers[0] if tiers else None})
    return rows


def advise(path: str, gpu: str = "b200", context: int = 32768, lanes: int = 8, world: int = 1) -> Dict:
    rec = recognise(path)
    out: Dict = {"path": path, "recognised": {k: v for k, v in rec.items() if k != "config"}}
    cfg: Optional[ModelConfig] = None
    if rec["kind"] == "hf":
        name = rec["config"].get("_name_or_path") or os.path.basename(os.path.normpath(path))
        try:
            desc = adapt_config(name, rec["config"])
        except AdaptError as e:
            out["verdict"] = f"refused: {e}"
            return out
        desc.pop("layer_table", None)
        out["description"] = desc
        out["gates"] = geometry_gates(desc, world, "bf16")
        cfg = match_registered(desc)
        if not desc.get("servable") or cfg is None:
            miss = desc.get("missing") or []
            out["verdict"] = ("not servable: the engine lacks " + ", ".join(miss)) if miss else \
                "not servable: no registered package has this geometry"
            return out
    elif rec["kind"] == "ninfer":
        base = rec["model_id"].split("@")[0]
        cfg = REGISTRY.get(base)
        if cfg is None:
            out["verdict"] = f"not servable: artifact model id '{rec['model_id']}' is not registered"
            return out
    elif rec["kind"] == "gguf":
        out["verdict"] = "convert first: `cli convert` reads the GGUF metadata and tensors and names the package"
        out["commands"] = [f"python -m ninfer_fusion_b200.cli convert {path} --out model.ninfer"]
        return out
    else:
        out["verdict"] = f"unknown: {rec.get('why', '')}"
        return out
    rows = fit(cfg, gpu, context, lanes, world)
    out["package"], out["gpu"], out["context"], out["lanes"], out["world"] = cfg.name, gpu, context, lanes, world
    out["fit"] = rows
    best = next((r for r in rows if r["weights"] == "bf16" and r["fits"]), None) or next((r for r in rows if r["fits"]), None)
    if best is None:
        # nothing fits resident: would it fit with part of the weights in pinned host memory, and at what price?
        from ..runtime.offload_budget import offload_verdict
        spec = GPUS[gpu]
        kv_values = 2 * len(cfg.attn_layers) * cfg.n_kv_heads * cfg.head_dim / world
        state = len(cfg.gdn_layers) * (cfg.gdn_v_heads * cfg.gdn_head_dim * cfg.gdn_head_dim * 4) / world
        kv = int(lanes * context * kv_values * KV_BITS["nvfp4"] / 8)
        small = min(rows, key=lambda r: r["weight_gib"])
        v = offload_verdict(int(small["weight_gib"] * (1 << 30)), kv, int(2 * lanes * state + 6 * (1 << 30)),
                            int(spec["mem_gib"] * (1 << 30)))
        out["offload"] = {"weights": small["weights"], "state": v.state, "offloaded_gib": round(v.offloaded_bytes / (1 << 30), 2),
                          "added_ms_per_round": round(v.added_ms_per_round, 1), "note": v.note}
        if v.state == "offload":
            keep = small["weight_gib"] - v.offloaded_bytes / (1 << 30)
            out["verdict"] = (f"fits one {gpu} only with weights off-loaded: {small['weights']} weights, nvfp4 KV, "
                              f"--weight-budget-gib {keep:.0f} (about {v.added_ms_per_round:.0f} ms more per decode round); "
                              f"sharding (--tp) avoids that price")
        else:
            out["verdict"] = (f"does not fit one {gpu} at {lanes} x {context} tokens in any weight format: shard it (--tp) "
                              f"or shorten the context")
        return out
    out["verdict"] = f"servable as {cfg.name}: {best['weights']} weights ({best['weight_gib']} GiB), {best['widest_kv']} KV"
    art = path if rec["kind"] == "ninfer" else "model.ninfer"
    cmds = [] if rec["kind"] == "ninfer" else [f"python -m ninfer_fusion_b200.cli convert {path} --out model.ninfer"]
    launch = "" if world == 1 else (f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {world} --master-addr 127.0.0.1 -m "
                                    f"ninfer_fusion_b200.cli")
    cmds.append((launch or "python -m ninfer_fusion_b200.cli") + f" serve --artifact {art} --device cuda --weights {best['weights']} "
                f"--kv-dtype {best['widest_kv']} --max-context {context} --max-lanes {lanes}" + (f" --tp {world}" if world > 1 else ""))
    out["commands"] = cmds
    return out
