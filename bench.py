#!/usr/bin/env python
"""Headline benchmark: decode tokens/s of the 27B-class hybrid decoder with fp8 KV.

    python bench.py --gpus N --steps K --warmup W

Config (BASELINE.json, second and third entries): 64 layers in a 3 GDN : 1 gated-GQA
pattern, hidden 5120, 24/4 heads of 256, GDN 16/48 heads of 128, FFN 17408, vocab 248320,
random-init bf16 weights, fp8-E4M3 per-row KV cache, batch 32, 2048-token uniform-random
prompts, greedy decode.  One "step" is one decode round of the whole batch.  N > 1 runs the
same model tensor-parallel over N ranks (strong scaling: the batch does not grow).

Timing: W untimed warm-up rounds, then exactly K rounds bracketed by barrier +
synchronize, timed with CUDA events on the launching stream, max over ranks.  The weights
(54 GB) are far larger than L2, so no explicit flush is needed between rounds.
`value` is the device-timed graph loop (token ids and positions advance on the device);
`e2e` runs the same K rounds through Generator.decode_step(): pinned-host descriptor -> one
H2D copy -> graph -> D2H of the sampled ids, every round.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_DECODE_TOK_S = 86.4  # reference, Qwen3.6-27B nvfp4, 7,680-token prompt, one RTX 5090 (docs/performance.md:537)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def reference_arm(args) -> int:
    """The reference arm: the reference's own Op benchmarks (its sources compiled unmodified for plain sm_100, see
    baseline/build_reference.sh) at the shapes of one 27B decode round, summed per round (baseline/reference_ops.py).

    The reference has no multi-GPU engine and no batched serving loop, and its model programs only start from
    artifact files that do not exist offline, so this is an Op sum, marked as such ("class": "op-sum").  On N GPUs
    it is what the reference could do with them: N independent replicas, each decoding batch / N sequences; the
    round time is the slowest replica's."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import reference_ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ["CUDA_VISIBLE_DEVICES"] = str(local)   # the bench mains use device 0 of what they see
    batch = max(1, args.batch // world)
    raw = os.environ.get("NFB_REFERENCE_RAW_DIR")
    res = reference_ops.run(T=batch, context=args.prompt_len, raw_dir=os.path.join(raw, f"rank{rank}") if raw else None)
    if "unavailable" in res:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": res["unavailable"]}))
        return 0
    sum_us = res["sum_us"]
    if world > 1:
        import torch
        import torch.distributed as dist
        dist.init_process_group("gloo")
        t = torch.tensor([sum_us], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sum_us = float(t[0])
        dist.destroy_process_group()
    if rank != 0:
        return 0
    if sum_us <= 0:
        print(json.dumps({"impl": "reference", "unavailable": "no reference Op benchmark produced a time on this device: "
                          + "; ".join(f"{r['op']}: {r.get('refused', '?')}" for r in res["rows"][:4])}))
        return 0
    ms = sum_us / 1e3
    print(json.dumps({
        "impl": "reference", "class": "op-sum",
        "metric": "decode tokens/sec/box + p50 TTFT at 1/2/4/8 B200, 27B hybrid fp8-KV",
        "value": round(batch * world / (ms / 1e3), 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (the reference benches' own generated operands)",
        "config": {"model": "qwen3.6-27b", "global_batch": batch * world, "seq_len": args.prompt_len,
                   "parallelism": "single" if world == 1 else f"{world} independent replicas of batch {batch}",
                   "kv": "fp8-e4m3-row", "weights": "bf16", "l2": "flushed between samples by the reference benches"},
        "note": "sum over the Ops of one decode round of (count per round x the median the reference's bench main printed); "
                "no launch gaps, no sampling loop, no host work: an optimistic round time for the reference",
        "ops": res["rows"], "missing": res["missing"]}))
    return 0


def speculative_run(args, cfg, device) -> int:
    """Draft-verify decoding against plain greedy decoding of the same model and prompts on one GPU: decode tok/s of
    both (device-timed, whole rounds, host round trips included), acceptance rate and
    tokens per round.  Prints one JSON line with class "speculative"."""
    import torch

    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.generator import Generator
    from ninfer_fusion_b200.runtime.speculative import SpeculativeGenerator

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print("bench.py: --spec runs on one GPU", file=sys.stderr)
        return 2
    B, L, Kd, R_ = args.batch, args.prompt_len, args.draft_tokens, args.tree_ranks
    n_rounds, warm = args.steps, max(3, args.warmup)
    weights = random_weights(cfg, device, seed=0, with_mtp=True, weight_format=args.weights)
    if args.spec == "dflash":
        from ninfer_fusion_b200.models.dflash import DFlashConfig, random_dflash_weights
        weights.update(random_dflash_weights(cfg, DFlashConfig(), weights, device))
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab, (L,), generator=g).tolist() for _ in range(B)]
    n_plain = (n_rounds + warm + 2) * (Kd + 1)
    max_ctx = L + n_plain + 64

    def timed(fn, n):
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1)

    plain = Generator(cfg, weights, device, max_batch=B, max_context=max_ctx, kv_format=args.kv_format, page_size=64,
                      prefill_chunk=2048, use_graph=True, pdl=bool(args.pdl))
    first = plain.prefill(prompts)
    stream = [[t] for t in first]
    for _ in range(warm):
        for b, t in enumerate(plain.decode_step()):
            stream[b].append(t)
    steps_plain = n_plain - warm - 1

    def plain_step():
        for b, t in enumerate(plain.decode_step()):
            stream[b].append(t)
    plain_ms = timed(plain_step, steps_plain)
    plain_tok_s = B * steps_plain / (plain_ms / 1e3)
    del plain
    torch.cuda.empty_cache()

    spec = SpeculativeGenerator(cfg, weights, device, max_batch=B, max_context=max_ctx, draft_tokens=Kd,
                                drafter=args.spec if args.spec in ("mtp", "dflash") else "hook", tree_ranks=R_,
                                kv_format=args.kv_format,
                                page_size=64, prefill_chunk=2048, pdl=bool(args.pdl), use_graph=not args.spec_eager,
                                adaptive_width=bool(args.adaptive_width),
                                draft_head_ids=list(range(args.draft_head)) if args.draft_head else None)
    if args.spec == "hook":
        # Synthetic drafts of mixed quality need the stream the VERIFY pass itself emits: with random-init weights many
        # logits are near ties, and a (K + 1)-row verify pass does not round like a one-row decode pass, so drafts copied
        # from the plain run above would be rejected for numerical reasons.  Record that stream first: rounds whose
        # drafts are all wrong emit exactly one token each, the verify pass's own.
        def wrong(b, history, k):
            return [(history[-1] + 1 + i) % cfg.vocab for i in range(k)]
        spec.draft_hook = wrong
        first_v = spec.prefill(prompts)
        stream = [[t] for t in first_v]
        for _ in range(n_plain - 1):
            for b, toks in enumerate(spec.decode_round()):
                stream[b].extend(toks)

        def hook(b, history, k):
            done = len(history) - L
            truth = stream[b][done:done + k]
            truth = truth + [0] * (k - len(truth))
            cut = (spec.rounds + b) % (k + 1)   # by round, not by position: a position rule locks into "all right"
            return [t if i < cut else (t + 1) % cfg.vocab for i, t in enumerate(truth)]
        spec.draft_hook = hook
        if R_ > 1:
            def tree_hook(b, history, k, r):
                # rank 0 = the chain's guess; when that guess is wrong, rank 1 holds the right token every other round,
                # so a side branch can rescue the depth; further ranks are wrong
                done = len(history) - L
                chain = hook(b, history, k)
                truth = stream[b][done:done + k] + [0] * k
                out_ = []
                for d in range(k):
                    row = [chain[d]]
                    for j in range(1, r):
                        rescue = j == 1 and chain[d] != truth[d] and done % 2 == 0
                        row.append(truth[d] if rescue else (truth[d] + 1 + j) % cfg.vocab)
                    out_.append(row)
                return out_
            spec.tree_hook = tree_hook
    spec.prefill(prompts)
    for _ in range(warm):
        spec.decode_round()
    e0, r0 = spec.emitted, spec.rounds
    spec_ms = timed(spec.decode_round, n_rounds)
    emitted = spec.emitted - e0
    spec.model.status.check("after speculative rounds")
    out = {
        "class": "speculative", "metric": "decode tokens/sec, draft-verify vs plain greedy (same model, prompts, GPU)",
        "value": round(emitted / (spec_ms / 1e3), 2), "unit": "tokens/s", "n_gpus": 1, "steps": n_rounds, "warmup": warm,
        "ms_per_step": round(spec_ms / n_rounds, 4), "higher_is_better": True, "dtype": args.weights,
        "data": "synthetic uniform-random token prompts, random-init weights",
        "config": {"model": cfg.name + ("" if not args.layers else " (SHRUNK: INVALID)"), "global_batch": B, "seq_len": L,
                   "kv": args.kv_format, "drafter": args.spec, "draft_tokens": Kd, "tree_ranks": R_,
                   "rounds": ("eager (no CUDA graph)" if not spec._graph_round_ok() else "one CUDA graph per round")
                   + ", one host round trip per round (accepted lengths and tokens)"},
        "draft_head_rows": args.draft_head or cfg.vocab,
        "adaptive_width": None if spec.width_ctl is None else {"width_now": spec.K, "decisions": spec.width_ctl.trace[-6:],
                                                                "cost_line_ms": spec.width_ctl.cost.fit()},
        "tokens_per_round": round(emitted / max(1, (spec.rounds - r0) * B), 3),
        "acceptance": round((emitted / max(1, (spec.rounds - r0) * B) - 1.0) / Kd, 4),
        "plain": {"tokens_per_s": round(plain_tok_s, 2), "ms_per_step": round(plain_ms / steps_plain, 4),
                  "rounds": "CUDA graph per round"},
        "speedup_vs_plain": round(emitted / (spec_ms / 1e3) / plain_tok_s, 3),
    }
    print(json.dumps(out), flush=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--kv-format", default="fp8")
    ap.add_argument("--model", default="qwen3.6-27b")
    ap.add_argument("--layers", type=int, default=0, help="debug only: shrink the layer count (result is marked invalid)")
    ap.add_argument("--no-ttft", action="store_true")
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--weights", default="bf16", choices=["bf16", "fp8", "nvfp4"],
                    help="matmul weight format (fp8 = e4m3 row-scale W8A8, nvfp4 = e2m1 block-scaled W4A4)")
    ap.add_argument("--experts", default="bf16", choices=["bf16", "fp8_block"],
                    help="routed expert format of MoE models (fp8_block = e4m3 with 128x128 block scales)")
    ap.add_argument("--emulate-tp-shard", type=int, default=0,
                    help="debug only: run ONE rank's 1/W shard of the tensor-parallel model on one GPU (no peers, so no "
                         "NVLink latency): the per-rank kernel chain of a W-GPU round (result is marked invalid)")
    ap.add_argument("--tp-mode", default="auto", choices=["auto", "fused", "oneshot", "nccl"],
                    help="tensor-parallel reduction: fused = reduce-scatter + all-gather inside the GEMMs, oneshot = "
                         "every rank receives every tile + one sum kernel, nccl = NCCL all-reduce baseline, auto = the "
                         "faster of fused / oneshot at this GPU count as measured (TensorParallel.best_mode)")
    ap.add_argument("--spec-eager", action="store_true", help="speculative rounds without CUDA graphs")
    ap.add_argument("--adaptive-width", action="store_true",
                    help="--spec: the draft width follows acceptance and measured round cost (ladder up to --draft-tokens)")
    ap.add_argument("--draft-head", type=int, default=0,
                    help="--spec mtp: propose from a shortlist head of this many LM-head rows (0 = the full head)")
    ap.add_argument("--spec", default="none", choices=["none", "mtp", "dflash", "hook"],
                    help="speculative decoding run (one GPU): mtp = the draft module proposes, dflash = the "
                         "block-diffusion draft model proposes the whole block in one pass (random-init "
                         "weights accept next to nothing), hook = synthetic drafts of mixed quality taken from the stream "
                         "the verify pass itself emits (the first (round + b) mod (K + 1) drafts right, the rest wrong)")
    ap.add_argument("--draft-tokens", type=int, default=4)
    ap.add_argument("--tree-ranks", type=int, default=1, help="candidates per depth of the draft tree (1 = chain)")
    ap.add_argument("--parallel", default="", choices=["", "tp", "ep"],
                    help="multi-GPU plan: tp = tensor parallel (dense default), ep = data parallel + expert parallel (MoE default)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    from ninfer_fusion_b200 import load_native
    from ninfer_fusion_b200.models.config import get_config
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.generator import Generator

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print("bench.py: launch with torch.distributed.run for --gpus > 1", file=sys.stderr)
            return 2
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    load_native()
    cfg = get_config(args.model)
    if args.layers:
        cfg = cfg.shrink(args.layers)
    comm = shard = None
    parallel = args.parallel or ("ep" if cfg.moe is not None else "tp")
    ep = world > 1 and parallel == "ep"
    if ep and (cfg.moe is None or args.batch % world):
        print("bench.py: --parallel ep needs a MoE model and a batch divisible by the GPU count", file=sys.stderr)
        return 2
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    if ep:
        # attention / GDN / router / shared expert replicated (same seed), routed experts: this rank's range only
        weights = random_weights(cfg, device, seed=0, expert_rank=rank, expert_world=world)
    elif world > 1:
        from ninfer_fusion_b200.parallel.tp import TensorParallel

        if args.tp_mode == "auto":
            args.tp_mode = TensorParallel.best_mode(world)
        comm = TensorParallel(cfg, rank, world, device, max_tokens=max(args.batch, 2048), mode=args.tp_mode)
        shard = comm.geometry
        weights = comm.random_shard_weights(seed=0)
        if args.weights == "bf16" and args.tp_mode == "fused":
            weights = comm.fold_norms(weights)   # layer norms become row scales of the gathered GEMMs
        if args.weights != "bf16":
            from ninfer_fusion_b200.models.weights import quantize_weights
            weights = quantize_weights(weights, args.weights)  # every rank quantises its own shard
    elif args.emulate_tp_shard > 1:
        from dataclasses import replace

        from ninfer_fusion_b200.parallel.tp import TensorParallel

        Wd = args.emulate_tp_shard
        cfg = replace(cfg, name=f"{cfg.name} (EMULATED 1/{Wd} SHARD: INVALID)", n_q_heads=cfg.n_q_heads // Wd,
                      n_kv_heads=max(1, cfg.n_kv_heads // Wd), gdn_qk_heads=cfg.gdn_qk_heads // Wd,
                      gdn_v_heads=cfg.gdn_v_heads // Wd, ffn_inter=cfg.ffn_inter // Wd, vocab=cfg.vocab // Wd)
        if args.tp_mode == "auto":
            args.tp_mode = "fused"
        comm = TensorParallel.loopback(cfg, 1, device, max_tokens=max(args.batch, 2048), mode=args.tp_mode)[0]
        shard = comm.geometry
        weights = random_weights(cfg, device, seed=0)
        if args.tp_mode == "fused":
            weights = comm.fold_norms(weights)
    else:
        weights = random_weights(cfg, device, seed=0, weight_format=args.weights)
    if args.weights != "bf16" and ep:
        print("bench.py: quantised weights are not wired for the expert-parallel plan", file=sys.stderr)
        return 2

    B, L, K, W = args.batch, args.prompt_len, args.steps, args.warmup
    if args.spec != "none":
        return speculative_run(args, cfg, device)
    B_local = B // world if ep else B  # expert parallel: every rank decodes its own share of the sequences
    max_ctx = L + 2 * (K + W) + 64
    gen = Generator(cfg, weights, device, max_batch=B_local, max_context=max_ctx, kv_format=args.kv_format,
                    page_size=64, prefill_chunk=2048, use_graph=True, pdl=bool(args.pdl), shard=shard, comm=comm)
    gen.model.expert_format = args.experts
    if ep:
        gen.model.ep = (rank, world, None)
    g = torch.Generator().manual_seed(1234 + (rank if ep else 0))
    prompts = [torch.randint(0, cfg.vocab, (L,), generator=g).tolist() for _ in range(B_local)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- TTFT: one 2048-token prompt, prefill to first token, p50 of 5 ----
    ttft_ms = None
    if not args.no_ttft:
        samples = []
        for i in range(6):
            barrier()
            t0 = time.perf_counter()
            gen.prefill(prompts[:1])
            torch.cuda.synchronize(device)
            samples.append((time.perf_counter() - t0) * 1e3)
        ttft_ms = statistics.median(samples[1:])

    # ---- batch prefill (untimed set-up of the decode state) ----
    barrier()
    t0 = time.perf_counter()
    gen.prefill(prompts)
    torch.cuda.synchronize(device)
    prefill_s = time.perf_counter() - t0

    # ---- device-timed decode: K graph replays, ids/positions advance on the device ----
    graph, finish = gen.decode_device_loop(W + K)
    for _ in range(W):
        graph.replay()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        graph.replay()
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    finish()
    gen.model.status.check("after device-timed decode")

    # ---- end to end through the public step API: H2D descriptors + graph + D2H ids per round ----
    for _ in range(W):
        gen.decode_step()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(K):
        gen.decode_step()
    e3.record()
    barrier()
    e2e_ms = e2.elapsed_time(e3)
    clocks = sampler.stop()
    gen.model.status.check("after end-to-end decode")

    t = torch.tensor([dev_ms, e2e_ms, ttft_ms or 0.0], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, ttft_max = (float(v) for v in t.tolist())
    if rank == 0:
        value = B * K / (dev_ms / 1e3)
        e2e_value = B * K / (e2e_ms / 1e3)
        launches = gen.model.ops.launches_last_forward * K
        # single-request decode tok/s of the reference on one RTX 5090 (docs/performance.md:537 and :318)
        baseline_tok_s = 271.1 if cfg.moe is not None else BASELINE_DECODE_TOK_S
        out = {
            "metric": "decode tokens/sec/box + p50 TTFT at 1/2/4/8 B200, 27B hybrid fp8-KV",
            "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None,
            "dtype": {"bf16": "bf16", "fp8": "fp8 e4m3 weights and activations, fp32 accumulate, bf16 residual",
                      "nvfp4": "nvfp4 weights and activations (block-scaled e2m1), fp32 accumulate, bf16 residual"}[args.weights],
            "data": "synthetic uniform-random token prompts, random-init weights",
            "config": {"model": cfg.name + ("" if not args.layers else " (SHRUNK: INVALID)"), "global_batch": B,
                       "seq_len": L, "parallelism": f"{parallel}{world}" if world > 1 else "single", "kv": args.kv_format + "-e4m3-row" if args.kv_format == "fp8" else args.kv_format,
                       "weights": args.weights if cfg.moe is None or args.experts == "bf16" else f"{args.weights} (routed experts {args.experts})",
                       "decode": "greedy, CUDA graph per round",
                       "l2": "inputs larger than L2 (all weights streamed every round), no flush",
                       "baseline_note": "no like-for-like published number: the reference documents single-request decode "
                                        f"on one RTX 5090 ({baseline_tok_s} tok/s), this line is a batch-{B} aggregate; "
                                        f"per sequence this run decodes {value / B:.1f} tok/s"},
            "ttft_ms_p50": round(ttft_max, 2) if ttft_ms is not None else None,
            "ttft_config": {"prompt_tokens": L, "batch": 1, "prefill_chunk": 2048},
            "batch_prefill_s": round(prefill_s, 3),
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms / K, 4),
                    "h2d_bytes_per_step": gen.bufs_decode.h2d_bytes(), "d2h_bytes_per_step": 4 * B_local},
            "gpu_launches": launches,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
