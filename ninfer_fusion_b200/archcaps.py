"""Architecture capability system: which instruction families the kernels of this package emit, which GPUs have
them, and which route (kernel) serves an (Op, format) pair on a given compute capability -- or the refusal that
names what is missing.

This package has ONE build target, sm_100a, so most of the table is refusals; it exists so that a wrong GPU, or an
artifact in a format without a route, is refused at load time with the missing capability by name instead of
failing inside a kernel launch.  Counterpart of the reference's capability bits, arch ladder, per-format floors and
route table (src/core/arch_caps.h:66-74,371-447, src/core/kernel_route.h `select_route`,
`require_artifact_formats_supported` in src/targets/registry.cpp:108-276); the rows here describe THIS package's
kernels, not the reference's.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple


class Cap(enum.IntFlag):
    """One bit per instruction family a kernel of this package needs (the asm it contains)."""
    NONE = 0
    MMA_SYNC_BF16 = 1 << 0        # mma.sync ... f32.bf16.bf16.f32 / f16 (attention for non-fp8 pages, GDN, vision, groupint)
    TMA_TENSOR = 1 << 1           # cp.async.bulk.tensor + mbarrier complete_tx
    CLUSTER_DSMEM = 1 << 2        # thread-block clusters, mapa / st.shared::cluster, barrier.cluster
    PDL = 1 << 3                  # griddepcontrol.wait / launch_dependents
    TCGEN05_F16 = 1 << 4          # tcgen05.mma kind::f16 with TMEM accumulators (bf16 GEMMs, MoE)
    TCGEN05_F8F6F4 = 1 << 5       # tcgen05.mma kind::f8f6f4 (fp8 W8A8 GEMMs, fp8 experts, fp8-page attention)
    TCGEN05_MXF4NVF4 = 1 << 6     # tcgen05.mma kind::mxf4nvf4.block_scale + tcgen05.cp of scale factors (nvfp4 W4A4)
    CVT_FP4 = 1 << 7              # cvt.rn.f16x2.e2m1x2 (nvfp4 KV pages)
    CVT_FP8 = 1 << 8              # cvt e4m3 <-> f16x2 (fp8 KV pages, quantisers)


@dataclass(frozen=True)
class ArchRung:
    sm: int            # major * 10 + minor, as torch.cuda.get_device_capability reports it
    label: str
    parts: str
    caps: Cap
    note: str


_AMPERE = Cap.MMA_SYNC_BF16
_HOPPER = _AMPERE | Cap.TMA_TENSOR | Cap.CLUSTER_DSMEM | Cap.PDL | Cap.CVT_FP8
_BLACKWELL_DC = _HOPPER | Cap.TCGEN05_F16 | Cap.TCGEN05_F8F6F4 | Cap.TCGEN05_MXF4NVF4 | Cap.CVT_FP4

ARCH_LADDER: Tuple[ArchRung, ...] = (
    ArchRung(80, "Ampere", "A100 / A30", _AMPERE, "no TMA, no clusters, no tcgen05: none of the GEMM routes exist"),
    ArchRung(86, "Ampere", "RTX 30xx / A10", _AMPERE, "as sm_80"),
    ArchRung(89, "Ada", "RTX 40xx / L40S", _AMPERE | Cap.CVT_FP8, "fp8 conversions, still no TMA / tcgen05"),
    ArchRung(90, "Hopper", "H100 / H200", _HOPPER,
             "TMA, clusters and programmatic launch exist, the tensor path is wgmma: tcgen05 kernels do not assemble"),
    ArchRung(100, "Blackwell data centre", "B200 (sm_100a)", _BLACKWELL_DC, "the build target of this package"),
    ArchRung(103, "Blackwell Ultra", "B300 (sm_103a)", _BLACKWELL_DC,
             "same instruction families; the library is built for sm_100a only, so it does not load there as built"),
    ArchRung(120, "Blackwell RTX", "RTX 50xx (sm_120a)", _HOPPER | Cap.CVT_FP4,
             "no tcgen05 / TMEM (its tensor path is mma.sync): none of the GEMM routes exist"),
)

BUILD_TARGET_SM = 100


def arch_rung(sm: int) -> Optional[ArchRung]:
    for r in ARCH_LADDER:
        if r.sm == sm:
            return r
    return None


class RouteRefused(ValueError):
    """No kernel of this package serves the request on this architecture; `missing` names the capabilities."""

    def __init__(self, message: str, missing: Cap = Cap.NONE):
        super().__init__(message)
        self.missing = missing


# (op, format) -> (route name = source file that implements it, capabilities it needs)
_ROUTES: Dict[Tuple[str, str], Tuple[str, Cap]] = {
    ("linear", "BF16"): ("csrc/gemm/gemm_bf16.cu", Cap.TMA_TENSOR | Cap.TCGEN05_F16 | Cap.CLUSTER_DSMEM | Cap.PDL),
    ("linear", "FP8_E4M3FN_ROW_BF16S"): ("csrc/gemm/gemm_quant.cu", Cap.TMA_TENSOR | Cap.TCGEN05_F8F6F4 | Cap.CLUSTER_DSMEM),
    ("linear", "NVFP4"): ("csrc/gemm/gemm_quant.cu", Cap.TMA_TENSOR | Cap.TCGEN05_MXF4NVF4 | Cap.CLUSTER_DSMEM),
    ("linear", "Q4G64_F16S"): ("csrc/gemm/gemm_groupint.cu", Cap.TMA_TENSOR | Cap.MMA_SYNC_BF16),
    ("linear", "Q5G64_F16S"): ("csrc/gemm/gemm_groupint.cu", Cap.TMA_TENSOR | Cap.MMA_SYNC_BF16),
    ("linear", "Q6G64_F16S"): ("csrc/gemm/gemm_groupint.cu", Cap.TMA_TENSOR | Cap.MMA_SYNC_BF16),
    ("linear", "W8G32_F16S"): ("csrc/gemm/gemm_groupint.cu", Cap.TMA_TENSOR | Cap.MMA_SYNC_BF16),
    ("experts", "BF16"): ("csrc/moe/moe_grouped_gemm.cu", Cap.TMA_TENSOR | Cap.TCGEN05_F16),
    ("experts", "FP8_E4M3FN_BLOCK128_F32S"): ("csrc/moe/moe_grouped_gemm_fp8.cu", Cap.TMA_TENSOR | Cap.TCGEN05_F8F6F4),
    ("decode_attention", "fp8"): ("csrc/attention/paged_attention_tc.cu", Cap.TMA_TENSOR | Cap.TCGEN05_F8F6F4 | Cap.CVT_FP8),
    ("decode_attention", "bf16"): ("csrc/attention/paged_attention_mma.cu", Cap.MMA_SYNC_BF16 | Cap.PDL),
    ("decode_attention", "int8"): ("csrc/attention/paged_attention_mma.cu", Cap.MMA_SYNC_BF16 | Cap.PDL),
    ("decode_attention", "nvfp4"): ("csrc/attention/paged_attention_mma.cu", Cap.MMA_SYNC_BF16 | Cap.CVT_FP4 | Cap.CVT_FP8),
    ("decode_attention", "mixed"): ("csrc/attention/paged_attention_mma.cu", Cap.MMA_SYNC_BF16 | Cap.CVT_FP4 | Cap.CVT_FP8),
    ("prefill_attention", "*"): ("csrc/attention/paged_attention_prefill.cu", Cap.MMA_SYNC_BF16 | Cap.PDL),
    ("gdn", "*"): ("csrc/gdn/gdn_recurrent.cu, gdn_chunked.cu", Cap.MMA_SYNC_BF16 | Cap.CLUSTER_DSMEM | Cap.PDL),
    ("tp_collectives", "*"): ("csrc/gemm/gemm_bf16.cu (kEpiRsAg), csrc/comm/tp_kernels.cu", Cap.TCGEN05_F16 | Cap.TMA_TENSOR),
}
_TEXT_FORMATS = ("FP32", "I32")   # small tensors read by pointwise kernels: no capability beyond a CUDA GPU


def caps_of(sm: int) -> Cap:
    r = arch_rung(sm)
    if r is None:
        raise RouteRefused(f"compute capability {sm // 10}.{sm % 10} has no row in the architecture ladder of this package "
                           f"({', '.join(f'sm_{x.sm}' for x in ARCH_LADDER)}): add the row with measured evidence first")
    return r.caps


def select_route(op: str, fmt: str, sm: int) -> str:
    """The source of the kernel that serves (`op`, `fmt`) on `sm`, or RouteRefused naming what is missing."""
    entry = _ROUTES.get((op, fmt)) or _ROUTES.get((op, "*"))
    if entry is None:
        raise RouteRefused(f"no kernel in this package implements {op} over {fmt}")
    route, need = entry
    have = caps_of(sm)
    missing = need & ~have
    if missing:
        names = ", ".join(c.name for c in Cap if c and c in missing)
        raise RouteRefused(f"{op} over {fmt} runs through {route}, which needs {names}; sm_{sm} "
                           f"({arch_rung(sm).label}) does not have {'it' if len(names.split(',')) == 1 else 'them'}", missing)
    if sm != BUILD_TARGET_SM:
        raise RouteRefused(f"{op} over {fmt}: sm_{sm} has the instruction families, but the native library is built for "
                           f"sm_{BUILD_TARGET_SM}a only")
    return route


def require_artifact_formats_supported(formats: Iterable[str], sm: int, experts: Iterable[str] = ()) -> List[str]:
    """Routes for every tensor format of an artifact (routed expert banks listed separately); raises RouteRefused for
    the first format without one.  Formats of small tensors (norm weights, tables) need no route."""
    routes = []
    for f in sorted(set(formats)):
        if f in _TEXT_FORMATS:
            continue
        routes.append(f"{f}: {select_route('linear', f, sm)}")
    for f in sorted(set(experts)):
        routes.append(f"experts {f}: {select_route('experts', f, sm)}")
    return routes


def device_report(sm: int) -> str:
    r = arch_rung(sm)
    if r is None:
        return f"sm_{sm}: not in the ladder"
    caps = ", ".join(c.name for c in Cap if c and c in r.caps) or "none"
    ok = "this package's build target" if sm == BUILD_TARGET_SM else "no route: " + r.note
    return f"sm_{sm} {r.label} ({r.parts}): {caps} -- {ok}"
