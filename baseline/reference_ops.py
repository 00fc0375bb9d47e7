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
    """(key, count per decode round, argv, note).  `T` = tokens per step (the decode batch).

    The reference batches its stateful Ops (GDN step, decode convolution, cached attention) over at most 8
    sequences (they exist for one request plus its draft tree), so a batch of T sequences is ceil(T / 8) calls of
    those; its bf16 Linear only accepts the weight shapes of its own models, so the GDN input projection is the
    three Linears it is made of there (z 6144, v 6144, q+k 4096 rows; the 96 gating rows have no bf16 bench shape and
    are left out).  Its fp8 benches are not part of the sum: `fp8_linear_swiglu` ended with
    "cudaErrorLaunchFailure: unspecified launch failure" on this GPU and is never started again."""
    t = str(T)
    lin = lambda n, k: ["linear", "--qtype", "BF16", "--n", str(n), "--k", str(k), "--t", t, "--warmup", "5", "--repeat", "30"]
    sb = min(T, 8)                       # sequences per call of a stateful Op
    calls = (T + sb - 1) // sb
    many = f"the Op takes at most 8 sequences: {calls} calls for {T}"
    return [
        ("gdn_in_proj_zv_bf16", 2 * N_GDN, lin(6144, 5120), "z and v rows of the GDN input projection (two Linears per layer)"),
        ("gdn_in_proj_qk_bf16", N_GDN, lin(4096, 5120), "q + k rows of the GDN input projection"),
        ("attn_in_proj_bf16", N_ATTN, ["attn_input_proj", "--format", "bf16", "--tokens", t, "--cache", "cold", "--warmup", "5",
                                       "--repeat", "30"], "q + gate + k + v rows 14336 x 5120, fused input projection"),
        ("out_proj_bf16_add", N_LAYERS, ["bf16_linear_add", "--t-sweep", t, "--route", "production", "--warmup", "5", "--repeat", "30"],
         "5120 x 6144 + residual (GDN out_proj and attention o_proj)"),
        ("mlp_gate_up_bf16", N_LAYERS, lin(34816, 5120), "gate and up rows, generic Linear (the SwiGLU product is a separate Op there, not timed)"),
        ("mlp_down_bf16", N_LAYERS, lin(5120, 17408), "down projection, generic Linear (the residual add is not timed)"),
        ("conv1d_silu", N_GDN * calls, ["causal_conv1d_silu", "--snapshot", "--batch", str(sb), "--tokens", "1", "--cache", "cold"],
         "decode step of the GDN convolution, batched snapshot form; " + many),
        ("gdn_step", N_GDN * calls, ["gated_delta_net", "--batch-update", "--batch", str(sb), "--warmup", "10", "--repeat", "40"],
         "recurrent update; " + many),
        ("rmsnorm_hidden", 2 * N_LAYERS + 1, ["rmsnorm", "--decode", "--kind", "hidden27", "--tokens", t], "input and post-attention norms"),
        ("attention_fp8", N_ATTN * T, ["causal_softmax_attention", "--entry", "cached", "--geometry", "d256-h24-kv4",
                                       "--kv-dtype", "fp8", "--batch", "1", "--tokens", "1", "--context", str(context),
                                       "--execution", "eager", "--cache", "cold", "--warmup", "5", "--repeat", "30"],
         f"decode attention over an fp8 cache: the `cached` entry takes one sequence, so a batch of {T} is {T} calls (the "
         "batched `append` entry needs the prefill objects, which do not fit the snapshot that travels to the GPU box)"),
        ("lm_head_bf16", 1, lin(248320, 5120), "vocabulary projection, generic Linear"),
        ("argmax", 1, ["argmax", "--shape", "full", "--cols", str(min(T, 128))], "greedy token choice"),
    ]


_MEDIAN = re.compile(r"median[=\s:]+\s*([0-9]+(?:\.[0-9]+)?)\s*us", re.I)
_US = re.compile(r"([0-9]+(?:\.[0-9]+)?)\s*us\b")


_LINEAR_ROW = re.compile(r"^(?:explicit|sweep)\s+\S+\s+\S+\s+\d+\s+\d+\s+\d+\s+([0-9]+(?:\.[0-9]+)?)", re.M)


def parse_median_us(text: str):
    """The first `median=... us` of the output, or the median_us column of the Linear bench's table row, else None
    (the raw text is kept beside it)."""
    m = _MEDIAN.search(text) or _LINEAR_ROW.search(text)
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
