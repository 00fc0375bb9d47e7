"""archkit: config adaptation, gates, GPU budget matrix."""
import json

import pytest

from ninfer_fusion_b200 import archkit
from ninfer_fusion_b200.archkit.adapt import AdaptError
from ninfer_fusion_b200.models.config import QWEN36_27B


def _qwen_hf():
    return {"text_config": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 24, "num_key_value_heads": 4,
                            "head_dim": 256, "partial_rotary_factor": 0.25, "rope_theta": 1e7, "full_attention_interval": 4,
                            "intermediate_size": 17408, "vocab_size": 248320, "hidden_act": "silu", "use_qk_norm": True,
                            "mtp_num_hidden_layers": 1}}


def test_adapt_hybrid_is_servable_and_complete():
    d = archkit.adapt_config("qwen3.6-27b", _qwen_hf())
    assert d["servable"] and d["missing"] == [] and (d["full"], d["gdn"], d["sliding"]) == (16, 48, 0)
    assert len(d["layer_table"]) == 64 and d["layer_table"][3]["rotary_dim"] == 64 and d["layer_table"][0]["kind"] == "gdn"
    assert archkit.geometry_gates(d, world=4) == [] and archkit.geometry_gates(d, world=8)   # 4 kv heads do not split 8 ways
    assert any("kv_heads" in g for g in archkit.geometry_gates(d, world=8))


def test_adapt_sliding_model_is_refused_with_reasons():
    hf = {"num_hidden_layers": 8, "hidden_size": 2560, "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 256,
          "layer_types": ["sliding_attention"] * 3 + ["full_attention"] + ["sliding_attention"] * 3 + ["full_attention"],
          "sliding_window": 512, "hidden_act": "gelu", "final_logit_softcapping": 30.0, "no_rope_layers_idx": [3, 7],
          "intermediate_size": 10240, "vocab_size": 131072}
    d = archkit.adapt_config("spark-x2.5-4b", hf)
    assert d["identifier"] == "spark_x2_5_4b" and not d["servable"]
    assert {"all-attention-schedule", "geglu-mlp", "logit-softcap", "nope-layers"} <= set(d["missing"])
    assert (d["sliding"], d["full"]) == (6, 2) and d["layer_table"][3]["rotary_dim"] == 0 and d["layer_table"][0]["window"] == 512
    # the failures a scaffold must not hide
    bad = dict(hf, layer_types=hf["layer_types"][:5])
    with pytest.raises(AdaptError, match="5 entries for 8 layers"):
        archkit.adapt_config("x", bad)
    with pytest.raises(AdaptError, match="not a known layer kind"):
        archkit.adapt_config("x", dict(hf, layer_types=["mamba"] * 8))
    with pytest.raises(AdaptError, match="sliding_window"):
        archkit.adapt_config("x", dict(hf, sliding_window=0))
    with pytest.raises(AdaptError, match="lacks hidden_size"):
        archkit.adapt_config("x", {"num_hidden_layers": 2})
    assert archkit.fold_identifier("4B-model.v2") == "m_4b_model_v2"


def test_gates_name_each_violation():
    d = {"head_dim": 512, "q_heads": 30, "kv_heads": 4, "hidden": 5000, "intermediate": 1000}
    g = archkit.geometry_gates(d, world=3, weight_format="nvfp4")
    text = " | ".join(g)
    for word in ("head_dim 512", "non-integer GQA", "hidden 5000", "kv_heads 4 % world 3", "intermediate 1000 % world 3", "nvfp4 scale tile"):
        assert word in text, (word, g)


def test_budget_matrix_orders_formats_and_tiers():
    rows = archkit.budget_matrix(QWEN36_27B, world=1, batch=8)
    by = {(r["gpu"], r["weights"]): r for r in rows}
    b = by[("b200", "bf16")]
    assert b["fits"] and 49 < b["weight_gib"] < 52 and 110 < b["decode_tok_s_roofline"] < 135
    assert by[("b200", "nvfp4")]["weight_gib"] < by[("b200", "fp8")]["weight_gib"] < b["weight_gib"]
    ctx = b["max_context"]
    assert ctx["nvfp4"] > ctx["fp8"] > ctx["bf16"] > 100000
    assert not by[("rtx5090", "bf16")]["fits"] and by[("rtx5090", "nvfp4")]["fits"]
    assert by[("rtx5090", "bf16")]["max_context"]["bf16"] == 0
    tp8 = {(r["gpu"], r["weights"]): r for r in archkit.budget_matrix(QWEN36_27B, world=4, batch=8)}
    assert tp8[("b200", "bf16")]["max_context"]["fp8"] > 4 * ctx["fp8"] * 0.9


def test_cli(tmp_path, capsys):
    from ninfer_fusion_b200.archkit.__main__ import main
    p = tmp_path / "config.json"
    p.write_text(json.dumps(_qwen_hf()))
    assert main(["adapt", "qwen3.6-27b", str(p), "--world", "2"]) == 0
    out = capsys.readouterr().out.splitlines()
    assert json.loads(out[0])["servable"] and len(json.loads(out[1])["layer_table"]) == 64
    assert main(["matrix", "--model", "tiny-dense"]) == 0
