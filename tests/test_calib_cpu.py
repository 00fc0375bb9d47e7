"""Context-cost calibration: the fit, the preset file and its refusals (measurements injected)."""
import json

import pytest

from ninfer_fusion_b200.runtime.planner import PRESETS, MaterializationPlanner, Owner
from ninfer_fusion_b200.utils import calib as C


def test_fit_recovers_a_known_line_and_scales_with_the_layer_ratio():
    cost = C.calibrate("box", lambda n: 0.002 + 45e-6 * n, lambda: 48.0, lambda: 5.5, layer_scale=8.0)
    assert cost.prefill_ns_per_token == pytest.approx(8 * 45_000.0, rel=1e-6)
    assert cost.prefill_fixed_ns == pytest.approx(8 * 2_000_000.0, rel=1e-6)
    assert (cost.host_gbps, cost.disk_gbps) == (48.0, 5.5)
    with pytest.raises(ValueError, match="does not grow"):
        C.calibrate("flat", lambda n: 0.01, lambda: 1.0, lambda: 1.0)
    with pytest.raises(ValueError, match="two"):
        C.fit_line([1.0], [1.0])


def test_preset_file_round_trip_and_refusals(tmp_path):
    cost = C.calibrate("box", lambda n: 0.001 + 30e-6 * n, lambda: 40.0, lambda: 4.0)
    path = tmp_path / "costs.json"
    path.write_text(C.to_json(cost, {"model": "tiny"}))
    back = C.load_preset(f"file:{path}")
    assert back == cost
    assert C.load_preset("b200") is PRESETS["b200"]
    with pytest.raises(ValueError, match="unknown planner preset"):
        C.load_preset("z9000")
    bad = json.loads(path.read_text())
    bad["host_gbps"] = 0
    path.write_text(json.dumps(bad))
    with pytest.raises(ValueError, match="host_gbps"):
        C.load_preset(f"file:{path}")
    path.write_text(json.dumps({"schema": "something else"}))
    with pytest.raises(ValueError, match="not a context-cost file"):
        C.load_preset(f"file:{path}")


def test_a_calibrated_preset_drives_the_planner(tmp_path):
    # slow host link, fast prefill: rebuilding a short frontier is cheaper than fetching it back
    cost = C.calibrate("odd", lambda n: 1e-6 * n + 1e-5, lambda: 0.05, lambda: 0.01)
    plan = MaterializationPlanner(cost).plan([Owner("short", pages=4, tokens=64, nbytes=64 << 20, hits=1)], need_pages=4)
    assert plan.complete and plan.actions["short"] == "drop"


def test_disk_probe_reads_what_it_wrote(tmp_path):
    assert C.disk_read_gbps(str(tmp_path), nbytes=8 << 20) > 0
    assert list(tmp_path.iterdir()) == []        # the scratch file is gone
