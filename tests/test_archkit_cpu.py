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


def test_model_import_recognises_judges_and_advises(tmp_path):
    from ninfer_fusion_b200 import cli
    from ninfer_fusion_b200.archkit import model_import as MI
    # a Hugging Face checkpoint directory of the 27B geometry (header-sized shards: nothing is loaded)
    hf = tmp_path / "Qwen3.6-27B"
    hf.mkdir()
    (hf / "config.json").write_text(json.dumps(_qwen_hf()))
    (hf / "model-00001-of-00002.safetensors").write_bytes(b"\0" * 64)
    (hf / "model-00002-of-00002.safetensors").write_bytes(b"\0" * 64)
    rec = MI.recognise(str(hf))
    assert rec["kind"] == "hf" and rec["shards"] == 2 and rec["bytes"] == 128
    adv = MI.advise(str(hf), gpu="b200", context=32768, lanes=8)
    assert adv["package"] == "qwen3.6-27b" and adv["verdict"].startswith("servable as qwen3.6-27b: bf16")
    assert adv["commands"][0].startswith("python -m ninfer_fusion_b200.cli convert") and "--kv-dtype" in adv["commands"][1]
    by = {r["weights"]: r for r in adv["fit"]}
    assert by["nvfp4"]["weight_gib"] < by["fp8"]["weight_gib"] < by["bf16"]["weight_gib"] and by["bf16"]["fits"]
    # a 32 GiB card: bf16 weights do not fit, a 4-bit format does, and the advice says so
    small = MI.advise(str(hf), gpu="rtx5090", context=8192, lanes=1)
    sby = {r["weights"]: r for r in small["fit"]}
    assert not sby["bf16"]["fits"] and sby["nvfp4"]["fits"] and "nvfp4" in small["verdict"] or "q4" in small["verdict"]
    # eight ranks: the launcher line and --tp
    tp = MI.advise(str(hf), gpu="b200", context=131072, lanes=8, world=8)
    assert "--nproc-per-node 8" in tp["commands"][-1] and tp["commands"][-1].endswith("--tp 8")
    # a geometry the engine does not serve is refused with what is missing
    odd = tmp_path / "other"
    odd.mkdir()
    (odd / "config.json").write_text(json.dumps({"num_hidden_layers": 8, "hidden_size": 2560, "num_attention_heads": 16,
                                                 "num_key_value_heads": 4, "head_dim": 256, "hidden_act": "gelu",
                                                 "intermediate_size": 10240, "vocab_size": 131072}))
    assert MI.advise(str(odd))["verdict"].startswith("not servable")
    # an artifact, a GGUF header, junk
    art = tmp_path / "t.ninfer"
    assert cli.main(["make-artifact", "--model", "tiny-dense", "--out", str(art)]) == 0
    a = MI.advise(str(art))
    assert a["recognised"]["kind"] == "ninfer" and a["package"] == "tiny-dense" and len(a["commands"]) == 1
    g = tmp_path / "m.gguf"
    g.write_bytes(b"GGUF" + (3).to_bytes(4, "little") + b"\0" * 8)
    assert MI.recognise(str(g)) == {"kind": "gguf", "version": 3, "bytes": 16} and MI.advise(str(g))["verdict"].startswith("convert first")
    junk = tmp_path / "x.bin"
    junk.write_bytes(b"hello")
    assert MI.advise(str(junk))["verdict"].startswith("unknown") and MI.recognise(str(tmp_path / "nope"))["kind"] == "unknown"
    from ninfer_fusion_b200.archkit.__main__ import main as archkit_main
    assert archkit_main(["import", str(hf)]) == 0 and archkit_main(["import", str(junk)]) == 1


def test_offload_budget_math_and_the_import_advice_that_uses_it(tmp_path):
    from ninfer_fusion_b200.archkit import model_import as MI
    from ninfer_fusion_b200.runtime.offload_budget import KvCapacityFit, KvCapacityPoint, offload_verdict
    fit = KvCapacityFit.from_points(KvCapacityPoint(1000, 10_000_000 + 4096, 16.0), KvCapacityPoint(4000, 20_000_000 + 4096, 8.0))
    assert fit.bytes_per_token_bit == pytest.approx(625.0) and fit.constant_bytes == pytest.approx(4096.0)
    assert fit.bytes_for(2000, 8.0) == pytest.approx(10_004_096.0)
    assert fit.bits_within(2000, 10_004_096) == pytest.approx(8.0) and fit.bits_within(0, 1) == 0.0
    with pytest.raises(ValueError):
        KvCapacityFit.from_points(KvCapacityPoint(1000, 1, 8.0), KvCapacityPoint(500, 2, 16.0))
    G = 1 << 30
    assert offload_verdict(50 * G, 20 * G, 5 * G, 80 * G).state == "resident"
    v = offload_verdict(50 * G, 40 * G, 5 * G, 80 * G, host_link_gbs=50.0)
    assert v.state == "offload" and v.offloaded_bytes == 15 * G and v.added_ms_per_round == pytest.approx(15 * G / 50e9 * 1e3)
    assert offload_verdict(50 * G, 80 * G, 5 * G, 80 * G).state == "does_not_fit"            # the KV leaves no room for the weights
    assert offload_verdict(50 * G, 40 * G, 5 * G, 80 * G, host_bytes=10 * G).state == "does_not_fit"
    # the import advice: 27B on a 32 GiB card at a long context fits only with off-loaded weights, and says what that costs
    hf = tmp_path / "Qwen3.6-27B"
    hf.mkdir()
    (hf / "config.json").write_text(json.dumps(_qwen_hf()))
    adv = MI.advise(str(hf), gpu="rtx5090", context=262144, lanes=4)
    assert adv["offload"]["state"] == "offload" and adv["offload"]["weights"] == "q4"
    if adv["offload"]["state"] == "offload":
        assert "--weight-budget-gib" in adv["verdict"] and adv["offload"]["added_ms_per_round"] > 0
