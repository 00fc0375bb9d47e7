"""Context-cost calibration: measures what the materialisation planner's cost model needs on THIS machine and writes
it as a preset file the CLI reads (`--planner file:<path>`).

    python -m ninfer_fusion_b200.utils.calib --model qwen3.6-27b --layers 8 --out b200_costs.json

Measured: (1) prefill time at several prompt lengths -> least-squares line `fixed + per_token * tokens` (the cost of
rebuilding a frontier by running its tokens again); (2) pinned-host <-> device copy rate over 256 MiB buffers (the
cost of restoring a frontier from the host tier); (3) sequential read rate of a scratch file (the disk tier).  A
layer-shrunk model scales the prefill line by n_layers / measured layers.  The measuring functions are injected, so
the fitting and file format are tested without a GPU.

Counterpart of the reference's context-cost calibration (bench/context_cost, tools/calib): its planner reads a
calibrated cost table instead of constants.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from typing import Callable, Dict, List, Sequence, Tuple

from ..runtime.planner import PRESETS, ContextCost

SCHEMA = "ninfer_context_cost_v1"


def fit_line(xs: Sequence[float], ys: Sequence[float]) -> Tuple[float, float]:
    """(intercept, slope) of the least-squares line through the points; intercept clamped at zero."""
    n = len(xs)
    if n < 2 or len(ys) != n:
        raise ValueError("need at least two (tokens, seconds) points")
    mx, my = sum(xs) / n, sum(ys) / n
    sxx = sum((x - mx) ** 2 for x in xs)
    if sxx == 0:
        raise ValueError("all prompt lengths are equal")
    slope = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sxx
    if slope <= 0:
        raise ValueError("prefill time does not grow with the prompt length: measurement is noise")
    return max(0.0, my - slope * mx), slope


def calibrate(name: str, prefill_s: Callable[[int], float], host_copy_gbps: Callable[[], float],
              disk_read_gbps: Callable[[], float], lengths: Sequence[int] = (512, 1024, 2048, 4096),
              layer_scale: float = 1.0) -> ContextCost:
    pts = [(n, prefill_s(n)) for n in lengths]
    fixed_s, per_tok_s = fit_line([p[0] for p in pts], [p[1] for p in pts])
    return ContextCost(name, per_tok_s * 1e9 * layer_scale, fixed_s * 1e9 * layer_scale, host_copy_gbps(), disk_read_gbps())


def to_json(cost: ContextCost, meta: Dict[str, object]) -> str:
    return json.dumps({"schema": SCHEMA, "name": cost.name, "prefill_ns_per_token": cost.prefill_ns_per_token,
                       "prefill_fixed_ns": cost.prefill_fixed_ns, "host_gbps": cost.host_gbps, "disk_gbps": cost.disk_gbps,
                       "copy_fixed_ns": cost.copy_fixed_ns, "measured": meta}, indent=1)


def load_preset(spec: str) -> ContextCost:
    """`b200` / `h100` / ... (built-in) or `file:<path>` written by this tool."""
    if spec.startswith("file:"):
        d = json.loads(open(spec[5:]).read())
        if d.get("schema") != SCHEMA:
            raise ValueError(f"{spec[5:]} is not a context-cost file ({SCHEMA})")
        for k in ("prefill_ns_per_token", "prefill_fixed_ns", "host_gbps", "disk_gbps"):
            if not isinstance(d.get(k), (int, float)) or d[k] < 0 or (k.endswith("gbps") and d[k] == 0):
                raise ValueError(f"{spec[5:]}: bad value for {k}")
        return ContextCost(str(d.get("name", "calibrated")), float(d["prefill_ns_per_token"]), float(d["prefill_fixed_ns"]),
                           float(d["host_gbps"]), float(d["disk_gbps"]), float(d.get("copy_fixed_ns", 20_000.0)))
    if spec not in PRESETS:
        raise ValueError(f"unknown planner preset '{spec}' (built in: {', '.join(sorted(PRESETS))}; or file:<path>)")
    return PRESETS[spec]


# ---- the measurements on a real machine ----
def _gpu_measurers(model: str, layers: int, device: str):
    import torch

    from ..models.config import get_config
    from ..models.weights import random_weights
    from ..runtime.generator import Generator
    cfg = get_config(model)
    full_layers = cfg.n_layers
    if layers:
        cfg = cfg.shrink(layers)
    w = random_weights(cfg, device, seed=0)
    gen = Generator(cfg, w, device, max_batch=1, max_context=8192 + 64, kv_format="fp8", page_size=64, prefill_chunk=2048,
                    use_graph=False)
    g = torch.Generator().manual_seed(0)

    def prefill_s(n: int) -> float:
        prompt = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist()]
        gen.prefill(prompt)                      # warm-up of this length (allocations, kernels)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        gen.prefill(prompt)
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    def host_copy_gbps() -> float:
        host = torch.empty(256 << 20, dtype=torch.uint8, pin_memory=True)
        dev = torch.empty_like(host, device=device)
        dev.copy_(host, non_blocking=True)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            dev.copy_(host, non_blocking=True)
            host.copy_(dev, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        return 8 * host.numel() / (e0.elapsed_time(e1) * 1e-3) / 1e9

    return prefill_s, host_copy_gbps, full_layers / cfg.n_layers


def disk_read_gbps(directory: str | None = None, nbytes: int = 256 << 20) -> float:
    with tempfile.NamedTemporaryFile(dir=directory, delete=False) as f:
        path = f.name
        f.write(os.urandom(1 << 20) * (nbytes >> 20))
        f.flush()
        os.fsync(f.fileno())
    try:
        t0 = time.perf_counter()
        with open(path, "rb", buffering=0) as f:
            while f.read(8 << 20):
                pass
        return nbytes / (time.perf_counter() - t0) / 1e9
    finally:
        os.unlink(path)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="qwen3.6-27b")
    ap.add_argument("--layers", type=int, default=8, help="measure a shrunken model and scale the line (0 = all layers)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--name", default="calibrated")
    ap.add_argument("--cold-dir", default=None, help="directory of the disk tier (default: the system scratch directory)")
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    prefill_s, host_gbps, scale = _gpu_measurers(a.model, a.layers, a.device)
    cost = calibrate(a.name, prefill_s, host_gbps, lambda: disk_read_gbps(a.cold_dir), layer_scale=scale)
    text = to_json(cost, {"model": a.model, "layers_measured": a.layers, "layer_scale": scale, "device": a.device})
    with open(a.out, "w") as f:
        f.write(text + "\n")
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
