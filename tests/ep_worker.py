"""Worker for the multi-GPU expert-parallel test (launched by torch.distributed.run).

Every rank builds the same full random weights, keeps the experts of its own range, and runs the
MoE block on its OWN tokens (a different count on every rank); the result must match the fp32
oracle of the whole expert set.  Then a tiny MoE model generates greedily, data-parallel with
expert-parallel MoE layers, eager and as a CUDA graph, against a single-GPU run.  Progress lines
are flushed; the last line starts with EP_OK or EP_FAIL.
"""
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ninfer_fusion_b200.models.config import TINY_MOE  # noqa: E402
from ninfer_fusion_b200.models.hybrid import HybridModel, Workspace  # noqa: E402
from ninfer_fusion_b200.models.moe import MoeBlock  # noqa: E402
from ninfer_fusion_b200.models.reference_model import ReferenceModel  # noqa: E402
from ninfer_fusion_b200.models.weights import random_weights  # noqa: E402
from ninfer_fusion_b200.ops import reference as R  # noqa: E402
from ninfer_fusion_b200.runtime.generator import Generator  # noqa: E402


def log(rank, msg):
    print(f"[rank {rank} {time.strftime('%H:%M:%S')}] {msg}", flush=True)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = TINY_MOE
    full = random_weights(cfg, dev, seed=3, std=0.05)
    ok, msgs = True, []

    # ---- block level: different token counts per rank ----
    model = HybridModel(cfg, full, dev, ep_rank=rank, ep_world=world)
    ws = Workspace(cfg, 256, 8, dev)
    model.moe = MoeBlock(cfg, dev, ws.max_tokens, rank, world)
    ref = ReferenceModel(cfg, full)
    p = "text/layers/1"
    nxt = full["text/layers/2/input_norm"]
    for step, base_T in enumerate((5, 40, 130)):
        T = base_T + 3 * rank
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        x0 = (torch.randn(T, cfg.hidden, device=dev, generator=g) * 0.5).bfloat16()
        h = torch.randn(T, cfg.hidden, device=dev, generator=g).bfloat16()
        ws.x[:T].copy_(x0)
        ws.normed[:T].copy_(h)
        model.moe.forward(model, ws, T, p, nxt, ws.normed[:T], global_tokens=world * (base_T + 3 * world))
        torch.cuda.synchronize()
        model.status.check()
        router = R.bf16_round(h.cpu().float() @ full[f"{p}/moe/router"].cpu().float().t())
        _, ids = R.moe_route(router[:, : cfg.moe.n_experts], cfg.moe.top_k, True)
        same = (model.moe.ids[:T].cpu().long() == ids).all(-1)
        want = R.bf16_round(x0.cpu().float() + ref._ffn(p, h.cpu().float()))
        err = (ws.x[:T].cpu().float() - want)[same].abs().max().item()
        tol = 0.02 * want.abs().max().item() + 0.02
        log(rank, f"block T={T}: max err {err:.4f} (tol {tol:.4f}), routed alike {same.float().mean():.3f}")
        if err > tol or same.float().mean().item() < 0.97:
            ok = False
            msgs.append(f"rank {rank} block T={T} err {err}")
        dist.barrier()

    # ---- model level: data parallel sequences, expert-parallel MoE ----
    torch.manual_seed(5)
    all_prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 33, 9, 20)]
    mine = all_prompts[rank::world]
    n_new = 8
    outs = {}
    for use_graph in (False, True):
        gen = Generator(cfg, full, dev, max_batch=4, max_context=256, kv_format="bf16", page_size=16,
                        prefill_chunk=64, use_graph=use_graph)
        gen.model.ep = (rank, world, None)
        gen.model.moe_global_tokens = world * 64
        outs[use_graph] = gen.generate(mine, n_new)
        torch.cuda.synchronize()
        gen.model.status.check()
        dist.barrier()
        log(rank, f"generate graph={use_graph}: {outs[use_graph][0][:6]}")
    single = Generator(cfg, full, dev, max_batch=4, max_context=256, kv_format="bf16", page_size=16,
                       prefill_chunk=64, use_graph=False).generate(mine, n_new)
    for use_graph, out in outs.items():
        for o, s in zip(out, single):
            n = 0
            while n < len(s) and o[n] == s[n]:
                n += 1
            if n < max(1, len(s) // 2):
                ok = False
                msgs.append(f"rank {rank} graph={use_graph}: {o} vs {s}")
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(("EP_OK" if int(flag.item()) == 1 else "EP_FAIL") + " " + "; ".join(msgs), flush=True)
    elif msgs:
        print("EP_FAIL " + "; ".join(msgs), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
