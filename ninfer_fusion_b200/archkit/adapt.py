"""Hugging Face config.json -> package description behind the capability gate."""
from __future__ import annotations

import re
from typing import Dict, List

from ..models import packages as PK


def fold_identifier(model_id: str) -> str:
    """'spark-x2.5-4b' -> 'spark_x2_5_4b': dots and dashes are not legal in generated identifiers."""
    out = re.sub(r"[^0-9a-zA-Z_]", "_", model_id.strip().lower())
    if not out or out[0].isdigit():
        out = "m_" + out
    return out


class AdaptError(ValueError):
    pass


_KIND_WORDS = {"full_attention": PK.FULL, "attention": PK.FULL, "global": PK.FULL,
               "sliding_attention": PK.SLIDING, "sliding": PK.SLIDING, "local": PK.SLIDING,
               "linear_attention": PK.GDN, "gated_delta_net": PK.GDN, "gdn": PK.GDN}


def _layer_kinds(cfg: Dict, n_layers: int) -> List[str]:
    types = cfg.get("layer_types")
    if types is not None:
        kinds = []
        for i, t in enumerate(types):
            if t not in _KIND_WORDS:
                raise AdaptError(f"layer_types[{i}] = '{t}' is not a known layer kind")
            kinds.append(_KIND_WORDS[t])
        return kinds
    interval = cfg.get("full_attention_interval")
    if interval:
        return [PK.FULL if (i + 1) % interval == 0 else PK.GDN for i in range(n_layers)]
    pattern = cfg.get("sliding_window_pattern")
    if pattern and cfg.get("sliding_window"):
        return [PK.FULL if (i + 1) % pattern == 0 else PK.SLIDING for i in range(n_layers)]
    return [PK.FULL] * n_layers


def adapt_config(model_id: str, hf: Dict) -> Dict:
    """Description of the model as the package table would hold it, plus the gate's verdict.  Raises AdaptError when
    the config cannot be turned into a complete layer table (the failure a scaffold must not paper over)."""
    cfg = hf.get("text_config", hf)
    try:
        n_layers, hidden = int(cfg["num_hidden_layers"]), int(cfg["hidden_size"])
        q_heads, kv_heads = int(cfg["num_attention_heads"]), int(cfg.get("num_key_value_heads", cfg["num_attention_heads"]))
    except KeyError as e:
        raise AdaptError(f"config.json lacks {e.args[0]}") from None
    head_dim = int(cfg.get("head_dim", hidden // q_heads))
    kinds = _layer_kinds(cfg, n_layers)
    if len(kinds) != n_layers:
        raise AdaptError(f"layer table has {len(kinds)} entries for {n_layers} layers")
    window = int(cfg.get("sliding_window") or 0)
    if PK.SLIDING in kinds and window <= 0:
        raise AdaptError("sliding layers without a sliding_window")
    rot = int(round(head_dim * float(cfg.get("partial_rotary_factor", 1.0))))
    theta = float(cfg.get("rope_theta", (cfg.get("rope_parameters") or {}).get("rope_theta", 10000.0)))
    nope = set(cfg.get("no_rope_layers_idx", []) or [])
    needs = {f"head-dim-{head_dim}"}
    n_gdn, n_full, n_slide = kinds.count(PK.GDN), kinds.count(PK.FULL), kinds.count(PK.SLIDING)
    if n_gdn:
        needs.add("gdn-hybrid-schedule")
        expect = [PK.FULL if (i + 1) % 4 == 0 else PK.GDN for i in range(n_layers)]
        if kinds != expect:
            needs.add("free-form-gdn-schedule")
    else:
        needs.add("all-attention-schedule")
    if n_slide:
        needs.add("sliding-window-attention")
    if nope:
        needs.add("nope-layers")
    if rot != head_dim:
        needs.add("partial-rope")
    if cfg.get("final_logit_softcapping"):
        needs.add("logit-softcap")
    if cfg.get("attn_logit_softcapping"):
        needs.add("attention-softcap")
    act = str(cfg.get("hidden_act", cfg.get("hidden_activation", "silu")))
    needs.add("swiglu-mlp" if act in ("silu", "swiglu") else "geglu-mlp")
    if cfg.get("num_experts") or cfg.get("num_local_experts"):
        needs.discard("swiglu-mlp")
        needs.add("sparse-moe")
    if cfg.get("use_qk_norm", cfg.get("qk_norm", False)):
        needs.add("qk-norm")
    if cfg.get("mtp_num_hidden_layers") or cfg.get("num_nextn_predict_layers"):
        needs.add("mtp-draft")
    table = []
    for i, k in enumerate(kinds):
        if k == PK.GDN:
            table.append({"layer": i, "kind": k})
        else:
            table.append({"layer": i, "kind": k, "rotary_dim": 0 if i in nope else rot, "rope_theta": 0.0 if i in nope else theta,
                          "window": window if k == PK.SLIDING else 0})
    missing = sorted(set(needs) - PK.ENGINE_CAPABILITIES)
    return {"model_id": model_id, "identifier": fold_identifier(model_id), "hidden": hidden, "layers": n_layers,
            "full": n_full, "sliding": n_slide, "gdn": n_gdn, "q_heads": q_heads, "kv_heads": kv_heads, "head_dim": head_dim,
            "intermediate": int(cfg.get("intermediate_size", 0)), "vocab": int(cfg.get("vocab_size", 0)),
            "needs": sorted(needs), "missing": missing, "servable": not missing, "layer_table": table}
