"""Worker for the pipeline-parallel test (launched by torch.distributed.run): every rank holds the full tiny model but
runs only its stage's layers; the greedy tokens must equal a single-GPU run.  The last line starts with PP_OK or PP_FAIL.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ninfer_fusion_b200.models.config import TINY_DENSE  # noqa: E402
from ninfer_fusion_b200.models.weights import random_weights  # noqa: E402
from ninfer_fusion_b200.parallel.pp import PipelineStage, StagePlan  # noqa: E402
from ninfer_fusion_b200.runtime.batch import SeqChunk  # noqa: E402
from ninfer_fusion_b200.runtime.generator import Generator  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = TINY_DENSE
    w = random_weights(cfg, dev, seed=7, std=0.05)
    torch.manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 40)]
    n_new = 8
    gen = Generator(cfg, w, dev, max_batch=2, max_context=256, kv_format="bf16", page_size=16, prefill_chunk=64, use_graph=False)
    want = gen.generate(prompts, n_new)          # single GPU, all layers
    gen.reset()

    plan = StagePlan.balanced(cfg.n_layers, world)
    # this rank keeps only its own stage's layer weights (plus embedding / head): a missing tensor would raise
    a, b = plan.stages[rank]
    keep = {k: v for k, v in w.items() if not k.startswith("text/layers/") or a <= int(k.split("/")[2]) < b}
    gen.model.w = keep
    stage = PipelineStage(gen.model, gen.ws, gen.kv, gen.states, plan, rank)
    B = len(prompts)
    slots = [gen.states.alloc() for _ in range(B)]
    for r in range(B):
        gen.kv.ensure(r, len(prompts[r]) + n_new + 1)
    gen.kv.publish()
    batch = gen.bufs_prefill.build([SeqChunk(r, slots[r], 0, prompts[r], True) for r in range(B)])
    ids = stage.step(batch)
    got = [[int(v)] for v in ids.tolist()]
    lengths = [len(p) for p in prompts]
    for _ in range(n_new - 1):
        batch = gen.bufs_decode.build([SeqChunk(r, slots[r], lengths[r], [got[r][-1]], True) for r in range(B)])
        ids = stage.step(batch)
        for r in range(B):
            got[r].append(int(ids[r]))
            lengths[r] += 1
    torch.cuda.synchronize()
    gen.model.status.check("pipeline run")
    ok = got == want
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(("PP_OK " if int(flag) else "PP_FAIL ") + f"stages {plan.spec()} got {got} want {want}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
