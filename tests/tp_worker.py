"""Worker for the multi-GPU tensor-parallel tests (launched by torch.distributed.run).

Every rank builds the same full random weights, takes its shard, generates greedily with the
fused peer-memory collectives (eager and CUDA graph) and with the NCCL baseline (eager), and
rank 0 compares against a single-GPU run of the same weights.  Progress lines are flushed so a
stall can be located; the last line starts with TP_OK or TP_FAIL.
"""
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ninfer_fusion_b200.models.config import TINY_DENSE  # noqa: E402
from ninfer_fusion_b200.models.weights import random_weights  # noqa: E402
from ninfer_fusion_b200.parallel.tp import TensorParallel  # noqa: E402
from ninfer_fusion_b200.runtime.generator import Generator  # noqa: E402


def log(rank, msg):
    print(f"[rank {rank} {time.strftime('%H:%M:%S')}] {msg}", flush=True)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = TINY_DENSE
    full = random_weights(cfg, dev, seed=7, std=0.05)
    torch.manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 70, 5)]
    n_new = 10
    results = {}
    for mode, use_graph in (("fused", False), ("fused", True), ("nccl", False)):
        log(rank, f"start {mode} graph={use_graph}")
        comm = TensorParallel(cfg, rank, world, dev, max_tokens=64, mode=mode)
        gen = Generator(cfg, comm.shard(full), dev, max_batch=4, max_context=256, kv_format="bf16", page_size=16,
                        prefill_chunk=64, use_graph=use_graph, shard=comm.geometry, comm=comm)
        results[(mode, use_graph)] = gen.generate(prompts, n_new)
        torch.cuda.synchronize()
        dist.barrier()
        log(rank, f"done {mode} graph={use_graph}: {results[(mode, use_graph)][0][:5]}")
    # quantised weights: shard first, quantise each shard; fused (peer-memory) and NCCL reductions must tell the same story
    from ninfer_fusion_b200.models.weights import quantize_weights
    qres, qlogits = {}, {}
    for fmt in ("nvfp4", "fp8"):
        for mode, use_graph in (("fused", True), ("nccl", False)):
            log(rank, f"start {fmt} {mode} graph={use_graph}")
            comm = TensorParallel(cfg, rank, world, dev, max_tokens=64, mode=mode)
            wq = quantize_weights(comm.shard(full), fmt)
            gen = Generator(cfg, wq, dev, max_batch=4, max_context=256, kv_format="bf16", page_size=16,
                            prefill_chunk=64, use_graph=use_graph, shard=comm.geometry, comm=comm)
            gen.prefill([prompts[0], prompts[2]])   # one ragged step (26 tokens): the logits of both last tokens stay in the workspace
            qlogits[(fmt, mode)] = gen.ws.logits[:2].float().clone()
            qres[(fmt, mode)] = gen.generate(prompts, n_new)
            torch.cuda.synchronize()
            gen.model.status.check()
            dist.barrier()
            log(rank, f"done {fmt} {mode}: {qres[(fmt, mode)][0][:5]}")
    ok = True
    msg = ""
    for fmt in ("nvfp4", "fp8"):
        # the two reductions differ only in rounding (fp32 partial tiles vs bf16 deltas); with 4-bit activations a
        # rounding difference can flip single codes downstream, so the logits are compared by direction and the
        # tokens only for fp8
        la, lb = qlogits[(fmt, "fused")], qlogits[(fmt, "nccl")]
        cos = torch.nn.functional.cosine_similarity(la, lb, dim=-1).min().item()
        msg += f" {fmt}: cos(fused, nccl) {cos:.4f};"
        if cos < (0.85 if fmt == "nvfp4" else 0.98):
            ok = False
        a, b = qres[(fmt, "fused")], qres[(fmt, "nccl")]
        if fmt == "fp8" and sum(int(x[0] == y[0]) for x, y in zip(a, b)) < len(a) - 1:
            ok = False
            msg += f" {fmt}: fused {a} vs nccl {b};"
        # every rank must hold the same tokens (the reductions are replicated, not approximate per rank)
        mine = torch.tensor(a, device=dev)
        ref0 = mine.clone()
        dist.broadcast(ref0, 0)
        if not torch.equal(mine, ref0):
            ok = False
            msg += f" {fmt}: rank {rank} diverged from rank 0;"
    if rank == 0:
        single = Generator(cfg, full, dev, max_batch=4, max_context=256, kv_format="bf16", page_size=16,
                           prefill_chunk=64, use_graph=False).generate(prompts, n_new)
        for key, out in results.items():
            # greedy decoding diverges for good after one near-tie flip (partial sums are reduced in a different
            # order than on one GPU), so compare the agreeing PREFIX of every sequence and the first token
            prefix = []
            for o, s in zip(out, single):
                n = 0
                while n < len(s) and o[n] == s[n]:
                    n += 1
                prefix.append(n)
            if min(prefix) < 1 or sum(prefix) < 0.5 * sum(len(s) for s in single):
                ok = False
            msg += f" {key}:prefix{prefix}"
        if results[("fused", False)] != results[("fused", True)]:
            ok = False
            msg += " fused graph!=eager"
    mine = torch.tensor(results[("fused", True)], device=dev)
    ref = mine.clone()
    dist.broadcast(ref, 0)
    if not torch.equal(mine, ref):
        print(f"TP_FAIL rank {rank} tokens differ from rank 0", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if not ok and rank != 0:
        print(f"TP_FAIL rank {rank}:{msg}", flush=True)
    ok = bool(int(flag.item()))
    dist.barrier()
    if rank == 0:
        print(("TP_OK" if ok else "TP_FAIL") + msg, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
