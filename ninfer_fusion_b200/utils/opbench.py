"""Per-op cold-cache micro-benchmarks with roofline fractions.

    python -m ninfer_fusion_b200.utils.opbench gemm --T 32 --N 34816 --K 5120 --epi swiglu
    python -m ninfer_fusion_b200.utils.opbench decode27b            # every decode GEMM of the 27B model
    python -m ninfer_fusion_b200.utils.opbench attn --batch 32 --ctx 2048 --kv fp8
    python -m ninfer_fusion_b200.utils.opbench gdn --batch 32

Each timed launch is preceded by a write of a buffer larger than L2 (256 MiB), timing
is CUDA events on the launching stream after warm-up, and achieved bytes / FLOPs
are divided by the MEASURED peaks in MEASURED_PEAKS.json at the repository root (6.65 TB/s
and 1.59 PFLOP/s if that file is absent).  Counterpart of the reference's bench/ops/*
(bench/README.md:215-233).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from .. import load_native
from ..ops import reference as R

EPI = {"store": 0, "residual": 1, "swiglu": 2, "partial": 3}


def measured_peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


class L2Flusher:
    def __init__(self):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.buf.fill_(1)


def time_op(fn, iters=20, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return statistics.median(ts), min(ts)


def bench_gemm(ops, T, N, K, epi, splits=0, iters=20, pdl=False):
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    e = EPI[epi]
    out_cols = N // 2 if epi == "swiglu" else N
    out = torch.empty((T, out_cols), dtype=torch.bfloat16, device="cuda")
    resid = torch.zeros((T, N), dtype=torch.bfloat16, device="cuda") if epi == "residual" else None
    part = None
    if epi == "partial":
        splits = splits or int(ops.gemm_pick_splits(T, N, K, 3))
        part = torch.empty(splits * T * N, device="cuda")
        normed = torch.empty((T, N), dtype=torch.bfloat16, device="cuda")
        nw = torch.zeros(N, dtype=torch.bfloat16, device="cuda")
        xres = torch.zeros((T, N), dtype=torch.bfloat16, device="cuda")

        def fn():
            ops.gemm_bf16(x, w, None, e, None, None, part, splits, status, pdl)
            ops.add_rmsnorm(part, splits, None, xres, xres, nw, normed, T, N, 1e-6, True, pdl)
    else:
        cl = splits if splits else int(ops.gemm_pick_splits(T, N, K, e))

        def fn():
            ops.gemm_bf16(x, w, out if e != 1 else resid, e, resid, None, None, cl, status, pdl)
    med, best = time_op(fn, iters=iters, flush=L2Flusher())
    assert int(status.item()) == 0, "kernel reported a bounded-wait failure"
    byts = N * K * 2 + T * K * 2 + T * out_cols * 2
    flops = 2.0 * T * N * K
    bw, fl, how = measured_peaks()
    return {"op": f"gemm_{epi}", "T": T, "N": N, "K": K, "splits": splits or 1, "us": round(med * 1e6, 2),
            "best_us": round(best * 1e6, 2), "GBps": round(byts / med / 1e9, 1), "TFLOPs": round(flops / med / 1e12, 1),
            "frac_hbm": round(byts / med / bw, 3), "frac_bf16": round(flops / med / fl, 3), "peaks": how}


def bench_groupint(ops, T, N, K, fmt, iters=20):
    """Streaming linear over groupwise-int codes (random codes, constant scales: timing only)."""
    from ..artifact import layouts as L
    from ..ops import groupint as G
    long_name = G.SHORT_NAMES[fmt]
    size = L.encoded_size(long_name, "row-split-k128-v1", (N, K))
    payload = torch.randint(0, 256, (size,), dtype=torch.uint8, device="cuda")
    group = L.GROUP_FORMATS[long_name][1]
    n_scale = N * (L.align_up(K, 128) // group)
    payload[size - 2 * n_scale:].copy_(torch.full((n_scale,), 0.01, dtype=torch.float16, device="cuda").view(torch.uint8))
    w = G.GroupIntWeight(long_name, payload, (N, K))
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    out = torch.empty((T, N), dtype=torch.bfloat16, device="cuda")
    med, best = time_op(lambda: G.linear(ops, x, w, out=out), iters=iters, flush=L2Flusher())
    byts = size + T * K * 2 + T * N * 2
    bw, _, how = measured_peaks()
    return {"op": f"groupint_{fmt}", "T": T, "N": N, "K": K, "us": round(med * 1e6, 2), "best_us": round(best * 1e6, 2),
            "GBps": round(byts / med / 1e9, 1), "frac_hbm": round(byts / med / bw, 3), "weight_MB": round(size / 1e6, 1),
            "peaks": how}


DECODE_27B = [("attn_in", 14336, 5120, "store"), ("gdn_in", 16480, 5120, "store"), ("gate_up", 34816, 5120, "swiglu"),
              ("o_proj", 5120, 6144, "partial"), ("down", 5120, 17408, "partial"), ("lm_head", 248320, 5120, "store")]


def bench_attn(ops, batch, ctx, kv, hq=24, hkv=4, D=256, P=64, iters=20, impl=0):
    fmt = R.KV_FORMAT_NAMES[kv]
    group = 64 if fmt == R.KV_INT8_GROUP else (16 if fmt == R.KV_NVFP4 else D)
    rb = 2 * D if fmt == R.KV_BF16 else (D // 2 if fmt == R.KV_NVFP4 else D)
    sb = {R.KV_BF16: 0, R.KV_FP8_ROW: 2, R.KV_INT8_GROUP: 2 * (D // group), R.KV_NVFP4: D // 16}[fmt]
    pages_per = (ctx + P - 1) // P
    n_pages = batch * pages_per
    k = torch.randint(0, 120, (n_pages, hkv, P, rb), dtype=torch.uint8, device="cuda")
    v = torch.randint(0, 120, (n_pages, hkv, P, rb), dtype=torch.uint8, device="cuda")
    ks = vs = None
    if sb:
        ks = torch.full((n_pages, hkv, P, sb), 0x20, dtype=torch.uint8, device="cuda")
        vs = torch.full((n_pages, hkv, P, sb), 0x20, dtype=torch.uint8, device="cuda")
    table = torch.randperm(n_pages, device="cuda").int().view(batch, pages_per)
    q = torch.randn(batch, hq, D, device="cuda").to(torch.bfloat16)
    from ..models.hybrid import pick_attention_split
    split, n_splits = pick_attention_split(ctx, batch * hkv, waves=8 if impl == 3 else 2)
    part_o = torch.empty(batch * hq * n_splits * D, device="cuda")
    part_ml = torch.empty(batch * hq * n_splits * 2, device="cuda")
    out = torch.empty((batch, hq * D), dtype=torch.bfloat16, device="cuda")
    seq = torch.arange(batch, dtype=torch.int32, device="cuda")
    lens = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")

    def fn():
        ops.paged_attention(q, hq, hkv, D, seq, lens, table, k, v, ks, vs, P, fmt, group, D ** -0.5, split, n_splits,
                            part_o, part_ml, None, out, None, None, impl, False)
    med, best = time_op(fn, iters=iters, flush=L2Flusher())
    byts = 2 * batch * ctx * hkv * (rb + sb)
    bw, _, how = measured_peaks()
    return {"op": "paged_attention", "impl": impl, "batch": batch, "ctx": ctx, "kv": kv, "split_keys": split, "n_splits": n_splits,
            "us": round(med * 1e6, 2), "GBps": round(byts / med / 1e9, 1), "frac_hbm": round(byts / med / bw, 3), "peaks": how}


def bench_gdn_prefill(ops, batch, tokens, hk=16, hv=48, iters=10):
    """conv1d + multi-token GDN recurrence over `tokens` tokens of `batch` sequences (the TTFT path)."""
    d = 128
    qk, vd = hk * d, hv * d
    C = 2 * qk + vd
    ld = C + vd + 2 * hv
    T = batch * tokens
    proj = (torch.randn(T, ld, device="cuda") * 0.5).to(torch.bfloat16)
    conv_w = (torch.randn(C, 4, device="cuda") * 0.3).to(torch.bfloat16)
    conv_state = torch.zeros((batch, 3, C), dtype=torch.bfloat16, device="cuda")
    ssm = torch.zeros((batch, hv, d, d), device="cuda")
    cu = (torch.arange(batch + 1, device="cuda") * tokens).to(torch.int32)
    tseq = torch.arange(batch, device="cuda").repeat_interleave(tokens).to(torch.int32)
    slot = torch.arange(batch, dtype=torch.int32, device="cuda")
    conv_out = torch.empty((T, C), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((T, vd), dtype=torch.bfloat16, device="cuda")
    A = torch.zeros(hv, device="cuda")
    nw = torch.ones(d, dtype=torch.bfloat16, device="cuda")
    res = {}
    chunk_ws = torch.empty(int(ops.gdn_chunked_workspace_bytes(T, batch, hv)), dtype=torch.uint8, device="cuda")
    for name, fn in (("conv1d", lambda: ops.causal_conv1d_silu(proj, 0, C, conv_w, cu, tseq, slot, conv_state, conv_out, True, False, False)),
                     ("gdn", lambda: ops.gdn_recurrent(conv_out, 0, qk, 2 * qk, proj, C, C + vd, C + vd + hv, hk, hv, A, A, nw, 1e-6,
                                                       cu, slot, ssm, True, out, False)),
                     ("gdn_chunked", lambda: ops.gdn_recurrent(conv_out, 0, qk, 2 * qk, proj, C, C + vd, C + vd + hv, hk, hv, A, A, nw,
                                                               1e-6, cu, slot, ssm, True, out, False, None, None, chunk_ws))):
        med, best = time_op(fn, iters=iters, flush=L2Flusher())
        res[name + "_us"] = round(med * 1e6, 1)
    ops.gdn_prefill_trace(True)
    ops.gdn_recurrent(conv_out, 0, qk, 2 * qk, proj, C, C + vd, C + vd + hv, hk, hv, A, A, nw, 1e-6, cu, slot, ssm, True, out, False)
    torch.cuda.synchronize()
    ph = ops.gdn_prefill_trace(False).tolist()
    res["phase_cycles(wait,prologue,serial,partial+barrier,epilogue)"] = ph
    res.update({"op": "gdn_prefill(conv, recurrence)", "batch": batch, "tokens": tokens, "heads": hv,
                "us_per_token": round(res["gdn_us"] / tokens, 4)})
    return res


def bench_gdn(ops, batch, hk=16, hv=48, iters=20):
    d = 128
    qk, vd = hk * d, hv * d
    C = 2 * qk + vd
    ld = C + vd + 2 * hv
    proj = (torch.randn(batch, ld, device="cuda") * 0.5).to(torch.bfloat16)
    conv_w = (torch.randn(C, 4, device="cuda") * 0.3).to(torch.bfloat16)
    conv_state = torch.zeros((batch, 3, C), dtype=torch.bfloat16, device="cuda")
    ssm = torch.zeros((batch, hv, d, d), device="cuda")
    cu = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
    seq = torch.arange(batch, dtype=torch.int32, device="cuda")
    conv_out = torch.empty((batch, C), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((batch, vd), dtype=torch.bfloat16, device="cuda")
    A = torch.zeros(hv, device="cuda")
    nw = torch.ones(d, dtype=torch.bfloat16, device="cuda")

    def fn():
        ops.causal_conv1d_silu(proj, 0, C, conv_w, cu, seq, seq, conv_state, conv_out, True, True, False)
        ops.gdn_recurrent(conv_out, 0, qk, 2 * qk, proj, C, C + vd, C + vd + hv, hk, hv, A, A, nw, 1e-6, cu, seq, ssm,
                          True, out, False)
    med, best = time_op(fn, iters=iters, flush=L2Flusher())
    byts = 2 * ssm.numel() * 4
    bw, _, how = measured_peaks()
    return {"op": "gdn_decode_step(conv+recurrent)", "batch": batch, "us": round(med * 1e6, 2),
            "GBps": round(byts / med / 1e9, 1), "frac_hbm": round(byts / med / bw, 3), "peaks": how}


def bench_vision(side_patches: int, layers: int, iters=5):
    """Full-geometry vision tower on one square image of side_patches x side_patches patches; also times the
    packed attention kernel alone and reports its FLOP rate."""
    import math
    from ..models import vision as V
    cfg = V.VisionConfig().scaled(layers, 5120)
    w = V.random_vision_weights(cfg, "cuda", seed=0)
    tower = V.VisionTower(cfg, w, "cuda")
    ctl = V.build_control([(1, side_patches, side_patches)])
    P = ctl.n_patches
    patches = (0.5 * torch.randn(P, cfg.patch_dim, device="cuda")).to(torch.bfloat16)
    med, best = time_op(lambda: tower.encode(patches, ctl), iters=iters, warmup=2)
    H = cfg.hidden
    gemm_flops = 2.0 * P * (cfg.patch_dim * H + layers * (3 * H * H + H * H + 2 * H * cfg.intermediate)) + \
        2.0 * (P / 4) * (cfg.merger_hidden ** 2 + cfg.merger_hidden * cfg.out_hidden)
    attn_flops = layers * 4.0 * P * P * H
    tiles = torch.from_numpy(V.attention_tiles(ctl.segments, tower.tile)).cuda()
    qkv = torch.randn(P, 3 * H, device="cuda").to(torch.bfloat16)
    out = torch.empty(P, H, device="cuda", dtype=torch.bfloat16)
    a_med, _ = time_op(lambda: tower.ops.packed_attention(qkv, out, tiles, cfg.heads, 1 / math.sqrt(cfg.head_dim)), iters=10)
    return {"op": "vision_tower", "patches": P, "layers": layers, "launches": tower.launches, "ms": round(med * 1e3, 3),
            "ms_best": round(best * 1e3, 3), "tflops": round((gemm_flops + attn_flops) / med / 1e12, 1),
            "attn_us": round(a_med * 1e6, 1), "attn_tflops": round(4.0 * P * P * H / a_med / 1e12, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "decode27b", "prefill27b", "attn", "gdn", "gdn_prefill", "vision", "groupint", "groupint1", "all"])
    ap.add_argument("--side", type=int, default=64, help="vision: patches per image side (64 = a 1024 x 1024 image)")
    ap.add_argument("--layers", type=int, default=27, help="vision: transformer blocks")
    ap.add_argument("--T", type=int, default=32)
    ap.add_argument("--N", type=int, default=34816)
    ap.add_argument("--K", type=int, default=5120)
    ap.add_argument("--epi", default="store", choices=list(EPI))
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--kv", default="fp8")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--pdl", type=int, default=0)
    ap.add_argument("--impl", type=int, default=0, help="attn: 1 = SIMT, 2 = mma.sync, 3 = tcgen05 (0 = all that apply)")
    a = ap.parse_args(argv)
    ops = load_native()
    rows = []
    if a.what == "gemm":
        rows.append(bench_gemm(ops, a.T, a.N, a.K, a.epi, a.splits, a.iters, bool(a.pdl)))
    if a.what in ("decode27b", "all"):
        for T in ([1, 32] if a.what == "all" else [a.T]):
            for name, N, K, epi in DECODE_27B:
                r = bench_gemm(ops, T, N, K, epi, 0, a.iters, bool(a.pdl))
                r["name"] = name
                rows.append(r)
    if a.what == "prefill27b":
        for name, N, K, epi in DECODE_27B[:5]:
            r = bench_gemm(ops, 2048, N, K, "residual" if epi == "partial" else epi, 0, max(3, a.iters // 4))
            r["name"] = name
            rows.append(r)
    if a.what in ("attn", "all"):
        for kv in (["bf16", "fp8", "int8", "nvfp4"] if a.what == "all" else [a.kv]):
            impls = [a.impl] if a.impl else ([1, 2, 3] if kv == "fp8" else [1, 2])   # 3 = tcgen05 (fp8-row pages)
            for impl in impls:
                rows.append(bench_attn(ops, a.batch, a.ctx, kv, iters=a.iters, impl=impl))
    if a.what in ("gdn", "all"):
        rows.append(bench_gdn(ops, a.batch, iters=a.iters))
    if a.what == "gdn_prefill":
        rows.append(bench_gdn_prefill(ops, a.batch, a.T, iters=a.iters))
        rows.append(bench_gdn_prefill(ops, a.batch, a.T, hk=2, hv=6, iters=a.iters))
    if a.what == "groupint1":
        rows.append(bench_groupint(ops, a.T, a.N, a.K, a.kv if a.kv in ("q4", "q5", "q6", "w8") else "q4", a.iters))
    if a.what == "groupint":
        for fmt in ("q4", "q6", "w8"):
            for T in (1, 8, 32):
                for name, N, K, _ in DECODE_27B[2:5]:
                    r = bench_groupint(ops, T, N, K, fmt, a.iters)
                    r["name"] = name
                    rows.append(r)
    if a.what == "vision":
        rows.append(bench_vision(a.side, a.layers, max(3, a.iters // 4)))
    for r in rows:
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
