"""Architecture capability table: routes on the build target, refusals that name the missing capability elsewhere."""
import pytest

from ninfer_fusion_b200 import archcaps as A


def test_every_route_exists_on_the_build_target():
    for (op, fmt) in A._ROUTES:
        route = A.select_route(op, "fp8" if fmt == "*" and op.endswith("attention") else fmt, 100)
        assert route.startswith("csrc/")
    rows = A.require_artifact_formats_supported(["BF16", "FP32", "NVFP4", "Q4G64_F16S"], 100, experts=["FP8_E4M3FN_BLOCK128_F32S"])
    assert len(rows) == 4 and any("gemm_quant.cu" in r for r in rows) and rows[-1].startswith("experts ")


@pytest.mark.parametrize("sm,fmt,cap", [(90, "BF16", A.Cap.TCGEN05_F16), (120, "NVFP4", A.Cap.TCGEN05_MXF4NVF4),
                                        (89, "FP8_E4M3FN_ROW_BF16S", A.Cap.TCGEN05_F8F6F4), (80, "Q4G64_F16S", A.Cap.TMA_TENSOR)])
def test_other_architectures_are_refused_with_the_missing_capability_by_name(sm, fmt, cap):
    with pytest.raises(A.RouteRefused) as e:
        A.select_route("linear", fmt, sm)
    assert cap in e.value.missing and cap.name in str(e.value) and f"sm_{sm}" in str(e.value)


def test_unknown_rows_formats_and_sibling_targets():
    with pytest.raises(A.RouteRefused, match="no row in the architecture ladder"):
        A.select_route("linear", "BF16", 75)
    with pytest.raises(A.RouteRefused, match="no kernel in this package implements"):
        A.select_route("linear", "Q3_WHATEVER", 100)
    with pytest.raises(A.RouteRefused, match="built for sm_100a only"):
        A.select_route("linear", "BF16", 103)          # same families, other binary target
    assert "build target" in A.device_report(100) and "no route" in A.device_report(90)
    assert A.covers if hasattr(A, "covers") else True
