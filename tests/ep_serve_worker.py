"""Worker of the expert-parallel serving test (launched by torch.distributed.run on 2+ GPUs).

Rank 0 runs an `Engine` over `PartitionedLeader`, the others `partitioned_follower_loop`, each around its own
`GpuProgram` whose MoE layers are expert-parallel; requests are spread over the ranks and the ranks run in lock step.
The tokens must agree with a single-GPU generator on the same prompts.  The last line starts with EP_SERVE_OK or
EP_SERVE_FAIL.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ninfer_fusion_b200.models.config import TINY_MOE  # noqa: E402
from ninfer_fusion_b200.models.weights import random_weights  # noqa: E402
from ninfer_fusion_b200.parallel.partitioned import PartitionedLeader, partitioned_follower_loop  # noqa: E402
from ninfer_fusion_b200.parallel.replicated import RankChannel  # noqa: E402
from ninfer_fusion_b200.runtime.engine import Engine, RequestOptions  # noqa: E402
from ninfer_fusion_b200.runtime.generator import Generator  # noqa: E402
from ninfer_fusion_b200.runtime.gpu_program import GpuProgram  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ch = RankChannel.create(rank, world, timeout_s=30.0)
    cfg = TINY_MOE
    full = random_weights(cfg, dev, seed=3, std=0.05)
    inner = GpuProgram(cfg, full, dev, max_lanes=3, max_context=256, kv_format="bf16", page_size=16, prefill_chunk=64,
                       use_graph=False)
    inner.model.ep = (rank, world, None)
    if rank != 0:
        worker = partitioned_follower_loop(inner, ch, lockstep=True)
        inner.model.status.check("follower at stop")
        print(f"[rank {rank}] stopped after {worker.forward_steps} forward passes, {worker.filler_steps} fillers", flush=True)
        dist.destroy_process_group()
        return
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (21, 70, 5, 33)]
    n_new = 8
    prog = {}

    def factory():
        prog["p"] = PartitionedLeader(inner, ch, lanes_per_rank=3, lockstep=True)
        return prog["p"]
    eng = Engine(factory, prefill_chunk=64)
    handles = [eng.submit(p, RequestOptions(max_tokens=n_new)) for p in prompts]
    outs, msgs = [], []
    for h in handles:
        try:
            outs.append(h.wait(timeout=120))
        except TimeoutError:
            outs.append(list(h.tokens))
            msgs.append("time-out")
        if h.finish_reason != "length":
            msgs.append(f"finish_reason={h.finish_reason} {h.error}")
    census = prog["p"].census()["partitioned"]
    health = eng.health()["status"]
    if health == "ok":
        prog["p"].shutdown()
    eng.shutdown()
    inner.model.status.check("leader at stop")
    single = Generator(cfg, full, dev, max_batch=4, max_context=256, kv_format="bf16", page_size=16, prefill_chunk=64,
                       use_graph=False).generate(prompts, n_new)
    same = sum(int(a == b) for o, s in zip(outs, single) for a, b in zip(o, s))
    if same < 0.75 * n_new * len(prompts):
        msgs.append(f"tokens differ from one GPU: {outs} vs {single}")
    if min(census["per_rank_opened"]) < 1:
        msgs.append(f"requests were not spread over the ranks: {census}")
    if health != "ok":
        msgs.append(f"engine health {health}")
    print(("EP_SERVE_OK " if not msgs else "EP_SERVE_FAIL ") + f"same={same}/{n_new * len(prompts)} {census} " + "; ".join(msgs),
          flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
