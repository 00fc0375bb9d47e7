"""Closed package table and its capability gate."""
import pytest

from ninfer_fusion_b200.models import packages as PK
from ninfer_fusion_b200.models.config import QWEN36_27B


def test_hybrid_family_is_served():
    for mid in ("qwen3.6-27b", "qwen3.6-35b-a3b", "qwen3.5-9b", "qwen3.8-27b", "tiny-dense", "tiny-moe"):
        cfg = PK.construct(mid)
        d = PK.describe(mid)
        assert d["servable"] and d["missing"] == [] and d["full"] + d["gdn"] == cfg.n_layers
    assert PK.construct("qwen3.6-27b") is QWEN36_27B
    d = PK.describe("qwen3.6-27b")
    assert (d["full"], d["gdn"], d["sliding"]) == (16, 48, 0)


def test_layer_tables_of_the_attention_only_packages():
    spark, muse, gemma = (PK.lookup(m) for m in ("spark-x2.5-4b", "muse-glimmer-30b", "gemma4-31b"))
    assert (spark.count(PK.SLIDING), spark.count(PK.FULL), spark.count(PK.GDN)) == (27, 9, 0)
    assert {l.window for l in spark.layers if l.kind == PK.SLIDING} == {512}
    assert {(l.rotary_dim, l.rope_theta) for l in spark.layers if l.kind == PK.FULL} == {(64, 5e6)}
    assert (muse.count(PK.SLIDING), muse.count(PK.FULL)) == (39, 13)
    assert all(l.rotary_dim == 0 for l in muse.layers if l.kind == PK.FULL)          # NoPE on the full layers
    assert muse.final_logit_softcap == 20.0
    assert (gemma.count(PK.SLIDING), gemma.count(PK.FULL)) == (50, 10)
    assert {l.head_dim for l in gemma.layers} == {256, 512}


def test_gate_refuses_and_names_what_is_missing():
    with pytest.raises(PK.PackageRefused, match="all-attention-schedule"):
        PK.construct("spark-x2.5-4b")
    with pytest.raises(PK.PackageRefused, match="nope-layers"):
        PK.construct("muse-glimmer-30b")
    with pytest.raises(PK.PackageRefused, match="head-dim-512"):
        PK.construct("gemma4-31b")
    with pytest.raises(PK.PackageRefused, match="unknown model id"):
        PK.construct("llama-7b")
    # an engine without MoE kernels refuses the MoE package, and only that one
    have = PK.ENGINE_CAPABILITIES - {"sparse-moe"}
    with pytest.raises(PK.PackageRefused, match="sparse-moe"):
        PK.construct("qwen3.6-35b-a3b", have)
    assert PK.construct("qwen3.6-27b", have) is QWEN36_27B
    # with every need granted the description-only packages are still not constructible
    everything = PK.ENGINE_CAPABILITIES | PK.lookup("spark-x2.5-4b").needs
    with pytest.raises(PK.PackageRefused, match="geometry description only"):
        PK.construct("spark-x2.5-4b", everything)
