"""Geometry and parallelism gates: the refusals a target must clear before weights are sharded or kernels launched."""
from __future__ import annotations

from typing import Dict, List


def geometry_gates(desc: Dict, world: int = 1, weight_format: str = "bf16") -> List[str]:
    """Violations (empty = pass) for a description from ``adapt_config`` or ``packages.describe`` with head counts."""
    out: List[str] = []
    hd, qh, kvh, hidden = desc.get("head_dim", 0), desc.get("q_heads", 0), desc.get("kv_heads", 0), desc.get("hidden", 0)
    inter = desc.get("intermediate", 0)
    if hd not in (128, 256):
        out.append(f"head_dim {hd}: the attention kernels are built for 128 and 256")
    if kvh and qh % kvh:
        out.append(f"query heads {qh} are not a multiple of kv heads {kvh} (non-integer GQA group)")
    if hidden % 128:
        out.append(f"hidden {hidden} is not a multiple of the 128-column GEMM tile")
    if world > 1:
        if kvh % world:
            out.append(f"kv_heads {kvh} % world {world} != 0: tensor parallelism splits KV heads whole")
        if inter and inter % world:
            out.append(f"intermediate {inter} % world {world} != 0: weight columns must split evenly")
        if hidden % (128 * world):
            out.append(f"hidden {hidden} is not a multiple of 128 x world: the reduce-scatter slices are 128-column tiles")
    if weight_format == "nvfp4":
        for name, n in (("hidden", hidden), ("intermediate", inter // max(1, world))):
            if n and n % 128:
                out.append(f"{name} shard {n} is not a multiple of the 128-row nvfp4 scale tile")
    return out
