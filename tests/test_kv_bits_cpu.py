"""K / V bit ceilings: joint, split (reconciled per layer, refused by index), ceiling mode, the score table."""
import pytest

from ninfer_fusion_b200.kv import kv_bits as KB
from ninfer_fusion_b200.kv.policy import build_ladder, parse_layer_storage


def test_joint_entry_and_its_refusals():
    plan = KB.entry_joint(16, 8.5)
    assert len(plan.tiers) == 16 and plan.avg_bits <= 8.5 + 1e-9
    assert parse_layer_storage(plan.spec, 16) == [t for t in plan.tiers]
    with pytest.raises(KB.KvBitsRefused, match="cheapest tier"):
        KB.entry_joint(16, 2.0)
    with pytest.raises(KB.KvBitsRefused, match="per-plane score table"):
        KB.entry_joint(16, 8.5, k_scores=KB.default_scores())
    assert KB.reachable_tiers(8.1) == ["nvfp4", "fp8"]


def test_equal_ceilings_reconcile_and_unequal_ones_are_refused_by_layer_index():
    same = KB.entry_split(12, 8.5, 8.5)
    assert same.tiers == same.k_tiers == same.v_tiers and same.spec == KB.entry_joint(12, 8.5).spec
    with pytest.raises(KB.KvBitsRefused) as e:
        KB.entry_split(12, 16.0, 4.5)
    assert e.value.layer == 0 and "layer 0: K wants bf16 and V wants nvfp4" in str(e.value)
    assert e.value.fallback is not None and e.value.fallback.avg_bits <= 4.5 + 1e-9     # the plan that honours both ceilings
    # a request that happens to land on the same tiers per layer deploys although the ceilings differ
    ok = KB.entry_split(8, 16.0, 16.5 - 0.5)
    assert ok.tiers == ["bf16"] * 8


def test_ceiling_mode_deploys_the_minimum_and_reports_the_headroom():
    p = KB.entry_split(10, 16.0, 8.5, mode="ceiling")
    assert p.k_tiers == p.v_tiers == p.tiers and p.k_avg_bits <= 8.5 + 1e-9
    assert set(p.headroom_bits) == {"k"} and p.headroom_bits["k"] == pytest.approx(16.0 - p.k_avg_bits, abs=1e-3)
    assert KB.entry_split(10, 8.5, 8.5, mode="ceiling").headroom_bits == {}
    with pytest.raises(KB.KvBitsRefused):
        KB.entry_split(10, 8.5, 8.5, mode="widen")


def test_resolution_of_the_front_end_flags():
    assert KB.resolve(6, bits=8.5).spec == KB.entry_joint(6, 8.5).spec
    assert KB.resolve(6, k_bits=8.5, v_bits=8.5).tiers == KB.entry_split(6, 8.5, 8.5).tiers
    for bad in (dict(), dict(bits=8.5, mode="split"), dict(bits=8.5, k_bits=8.5, v_bits=8.5), dict(k_bits=8.5),
                dict(k_bits=8.5, v_bits=8.5, mode="joint")):
        with pytest.raises(KB.KvBitsRefused):
            KB.resolve(6, **bad)


def test_score_table_round_trip_and_per_plane_tables(tmp_path):
    prior = KB.default_scores()
    text = KB.emit_scores(prior)
    back = KB.parse_scores(text, "roundtrip")
    assert back.penalties == prior.penalties and "provenance: prior" in text
    # a measured table that says fp8 is as good as bf16 moves the allocation of that plane only
    good_fp8 = KB.ScoreTable(dict(prior.penalties, fp8=0, int8=500), "measured.txt")
    base = KB.entry_split(8, 12.0, 12.0)
    tilted = KB._plane(8, 12.0, good_fp8, None)
    assert tilted.tiers.count("fp8") > base.k_tiers.count("fp8")
    with pytest.raises(KB.KvBitsRefused):                         # the two planes now want different tiers somewhere
        KB.entry_split(8, 12.0, 12.0, k_scores=good_fp8)
    both = KB.entry_split(8, 12.0, 12.0, scores=good_fp8)         # the common table is each plane's fall-back
    assert both.k_tiers == both.v_tiers == tilted.tiers
    for bad in ("fp8", "fp8=x", "fp8=1\nfp8=2", "# nothing\n"):
        with pytest.raises(ValueError):
            KB.parse_scores(bad)
    with pytest.raises(ValueError, match="does not have"):
        KB.ScoreTable({"rk4v4": 5}).apply(build_ladder())
    path = tmp_path / "scores.txt"
    assert KB.main(["score-table", f"emit={path}"]) == 0 and KB.parse_scores(path.read_text()).penalties == prior.penalties
    assert KB.main(["plan", "--layers", "4", "--kv-k-bits", "16", "--kv-v-bits", "4.5"]) == 2
    assert KB.main(["plan", "--layers", "4", "--kv-bits", "8.5", "--kv-tier-scores", str(path)]) == 0
