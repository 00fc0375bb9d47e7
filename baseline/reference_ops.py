"""Runs the reference's own Op benchmarks (built unmodified for plain sm_100 by build_reference.sh into
baseline/_ref/bin/ninfer_ref_benches) at the shapes of one 27B decode round and sums them into a per-round estimate.

This is the reference arm of bench.py.  The reference has no multi-GPU engine, no batched serving loop and no
bf16-weight model program that could be started without its artifact files, so the comparison is per Op: every
number below is printed by the reference's bench mains (their timing loops, their L2 flush, their median), and the
only arithmetic done here is  sum(count_per_round x median_us).  Rows the reference cannot run on this device (a route
whose objects did not build for sm_100, a batch its Op does not accept) are listed with the reason, never estimated.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BIN = HERE / "_ref" / "bin" / "ninfer_ref_benches"

# 27B hybrid: 48 gated-delta-net layers + 16 full-attention layers, hidden 5120, FFN 17408, vocab 248320
N_GDN, N_ATTN, N_LAYERS = 48, 16, 64


def commands(T: int, context: int):
    """(key, count per decode round, argv, note).  `T` = tokens per step (the decode batch)."""
    t = str(T)
    lin = lambda n, k: ["linear", "--qtype", "BF16", "--n", str(n), "--k", str(k), "--t", t, "--warmup", "5", "--repeat", "30"]
    gdn_batch = min(T, 8)
    return [
        ("gdn_in_proj_bf16", N_GDN, lin(16384, 5120), "qkv 10240 + z 6144 rows, bf16 weights, generic Linear"),
        ("gdn_ab_proj_bf16", N_GDN, lin(96, 5120), "a / b gating rows"),
        ("attn_in_proj_bf16", N_ATTN, ["attn_input_proj", "--format", "bf16", "--tokens", t, "--cache", "cold", "--warmup", "5",
                                       "--repeat", "30"], "q + gate + k + v rows 14336 x 5120, fused input projection"),
        ("out_proj_bf16_add", N_LAYERS, ["bf16_linear_add", "--t-sweep", t, "--route", "production", "--warmup", "5", "--repeat", "30"],
         "5120 x 6144 + residual (GDN out_proj and attention o_proj)"),
        ("mlp_gate_up_bf16", N_LAYERS, lin(34816, 5120), "gate and up rows, generic Linear (the SwiGLU product is a separate Op there)"),
        ("mlp_down_bf16", N_LAYERS, lin(5120, 17408), "down projection, generic Linear"),
        ("mlp_gate_up_fp8_swiglu", 0, ["fp8_linear_swiglu", "--t-sweep", t, "--warmup", "5", "--repeat", "30"],
         "fp8 weights, fused SwiGLU (context: the reference's fused form exists for quantised weights only)"),
        ("mlp_down_fp8_add", 0, ["fp8_linear_add", "--k", "17408", "--t-sweep", t, "--warmup", "5", "--repeat", "30"], "fp8 weights"),
        ("conv1d_silu", N_GDN, ["causal_conv1d_silu", "--decode", "--batch", t, "--cache", "cold"], "decode step of the GDN convolution"),
        ("gdn_step", N_GDN * ((T + gdn_batch - 1) // gdn_batch),
         ["gated_delta_net", "--batch-update", "--batch", str(gdn_batch), "--warmup", "10", "--repeat", "40"],
         f"recurrent update; the Op accepts batches up to 8, so a batch of {T} is {(T + gdn_batch - 1) // gdn_batch} calls"),
        ("rmsnorm_hidden", 2 * N_LAYERS + 1, ["rmsnorm", "--decode", "--kind", "hidden27", "--tokens", t], "input and post-attention norms"),
        ("attention_fp8", N_ATTN, ["causal_softmax_attention", "--entry", "cached", "--geometry", "d256-h24-kv4", "--kv-dtype", "fp8",
                                   "--batch", t, "--tokens", "1", "--context", str(context), "--execution", "eager", "--cache", "cold",
                                   "--warmup", "5", "--repeat", "30"], "decode attention over an fp8 cache"),
        ("lm_head_bf16", 1, lin(248320, 5120), "vocabulary projection, generic Linear"),
        ("argmax", 1, ["argmax", "--shape", "full", "--cols", str(min(T, 128))], "greedy token choice"),
    ]


_MEDIAN = re.compile(r"median[=\s:]+\s*([0-9]+(?:\.[0-9]+)?)\s*us", re.I)
_US = re.compile(r"([0-9]+(?:\.[0-9]+)?)\s*us\b")


def parse_median_us(text: str):
    """The first `median=... us` of the output, else None (the raw text is kept beside it)."""
    m = _MEDIAN.search(text)
    return float(m.group(1)) if m else None


def run(T: int = 32, context: int = 2048, raw_dir: str | None = None, timeout: int = 180):
    if not BIN.exists():
        return {"unavailable": f"{BIN.relative_to(HERE.parent)} is missing: run baseline/build_reference.sh"}
    rows, total, missing = [], 0.0, []
    for key, count, argv, note in commands(T, context):
        try:
            r = subprocess.run([str(BIN)] + argv, capture_output=True, text=True, timeout=timeout)
            out, rc = r.stdout + r.stderr, r.returncode
        except subprocess.TimeoutExpired:
            out, rc = "timed out", -1
        if raw_dir:
            os.makedirs(raw_dir, exist_ok=True)
            Path(raw_dir, f"{key}_T{T}.txt").write_text("$ ninfer_ref_benches " + " ".join(argv) + f"\n[rc {rc}]\n" + out)
        us = parse_median_us(out) if rc == 0 else None
        row = {"op": key, "per_round": count, "median_us": us, "note": note}
        if us is None:
            row["refused"] = (out.strip().splitlines() or ["no output"])[-1][:200]
            if count:
                missing.append(key)
        elif count:
            total += count * us
        rows.append(row)
    return {"T": T, "context": context, "rows": rows, "sum_us": round(total, 1), "missing": missing}


if __name__ == "__main__":
    T = int(sys.argv[1]) if len(sys.argv) > 1 else 32
    print(json.dumps(run(T, raw_dir=sys.argv[2] if len(sys.argv) > 2 else None), indent=1))
