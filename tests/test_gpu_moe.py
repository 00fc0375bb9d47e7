"""Sparse-MoE block (route, dispatch, grouped tcgen05 GEMMs, fused return, combine) against the fp32 oracle."""
import pytest
import torch

from ninfer_fusion_b200.models.config import TINY_MOE, ModelConfig, MoEConfig
from ninfer_fusion_b200.models.hybrid import HybridModel, Workspace
from ninfer_fusion_b200.models.moe import MoeBlock
from ninfer_fusion_b200.models.reference_model import ReferenceModel, ReferenceSequence
from ninfer_fusion_b200.models.weights import random_weights
from ninfer_fusion_b200.ops import reference as R
from ninfer_fusion_b200.runtime.generator import Generator

pytestmark = pytest.mark.gpu

MID_MOE = ModelConfig(
    name="mid-moe", n_layers=4, hidden=512, vocab=1024, n_q_heads=8, n_kv_heads=1, head_dim=256, rot_dim=64,
    rope_theta=1e7, gdn_qk_heads=2, gdn_v_heads=4, ffn_inter=0,
    moe=MoEConfig(n_experts=64, top_k=8, expert_inter=256, shared_inter=128), max_context=4096)


@pytest.mark.parametrize("cfg", [TINY_MOE, MID_MOE], ids=lambda c: c.name)
@pytest.mark.parametrize("T", [1, 7, 33, 200, 700])
def test_moe_block_matches_oracle(cfg, T):
    torch.manual_seed(T)
    w = random_weights(cfg, "cuda", seed=3, std=0.05)
    model = HybridModel(cfg, w, "cuda")
    ws = Workspace(cfg, 1024, 8, "cuda")
    p = "text/layers/1"
    x0 = (torch.randn(T, cfg.hidden, device="cuda") * 0.5).bfloat16()
    h = torch.randn(T, cfg.hidden, device="cuda").bfloat16()
    ws.x[:T].copy_(x0)
    ws.normed[:T].copy_(h)
    nxt = w["text/layers/2/input_norm"]
    model.moe = MoeBlock(cfg, "cuda", ws.max_tokens)
    for rep in range(2):  # second call exercises the counters' second epoch
        ws.x[:T].copy_(x0)
        ws.normed[:T].copy_(h)
        model.moe.forward(model, ws, T, p, nxt, ws.normed[:T])
        torch.cuda.synchronize()
        model.status.check()
    ref = ReferenceModel(cfg, {k: v.cpu() for k, v in w.items()})
    # routing is exact up to bf16 rounding of the logits (a near-tie may swap the last expert)
    router = R.bf16_round(h.cpu().float() @ w[f"{p}/moe/router"].cpu().float().t())
    wts, ids = R.moe_route(router[:, : cfg.moe.n_experts], cfg.moe.top_k, True)
    got_ids = model.moe.ids[:T].cpu().long()
    same = (got_ids == ids).all(-1)
    assert same.float().mean().item() >= 0.98
    assert torch.allclose(model.moe.weights[:T].cpu()[same], wts[same], atol=2e-3)
    ffn = ref._ffn(p, h.cpu().float())
    want_x = R.bf16_round(x0.cpu().float() + ffn)
    got_x = ws.x[:T].cpu().float()
    scale = want_x.abs().max().item()
    assert (got_x - want_x)[same].abs().max().item() <= 0.02 * scale + 0.02
    want_n = R.rmsnorm(want_x, nxt.cpu().float(), cfg.rms_eps, True)
    got_n = ws.normed[:T].cpu().float()
    assert (got_n - want_n)[same].abs().max().item() <= 0.03 * want_n.abs().max().item() + 0.03


def test_moe_greedy_generation_matches_reference():
    cfg = TINY_MOE
    w = random_weights(cfg, "cuda", seed=11, std=0.05)
    gen = Generator(cfg, w, "cuda", max_batch=4, max_context=512, kv_format="bf16", page_size=16, prefill_chunk=64,
                    use_graph=True)
    ref = ReferenceModel(cfg, {k: v.cpu() for k, v in w.items()})
    torch.manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 70, 5)]
    n_new = 10
    out = gen.generate(prompts, n_new)
    agree = total = 0
    for b, p in enumerate(prompts):
        seq = ReferenceSequence(cfg, R.KV_BF16)
        hid = ref.forward(seq, torch.tensor(p))
        for j in range(n_new):
            lg = ref.logits(hid[-1:])[0]
            top2 = lg.topk(2).values
            if (top2[0] - top2[1]).item() > 0.05:
                total += 1
                agree += int(int(R.argmax_lowest(lg[None])[0]) == out[b][j])
            hid = ref.forward(seq, torch.tensor([out[b][j]]))
    assert total > 8 and agree / total >= 0.9, f"{agree}/{total}"


@pytest.mark.parametrize("cfg", [TINY_MOE, MID_MOE], ids=lambda c: c.name)
@pytest.mark.parametrize("T", [3, 40, 300])
def test_moe_block_fp8_block_scaled_experts(cfg, T):
    """Routed experts as e4m3 with 128x128 block scales (two-level accumulation kernel) against an oracle that uses
    the de-quantised expert weights and the same per-row / per-128 activation quantisation."""
    from ninfer_fusion_b200.ops import quant as Q
    torch.manual_seed(T)
    w = random_weights(cfg, "cuda", seed=3, std=0.05)
    model = HybridModel(cfg, w, "cuda")
    ws = Workspace(cfg, 512, 8, "cuda")
    p = "text/layers/1"
    m = cfg.moe
    x0 = (torch.randn(T, cfg.hidden, device="cuda") * 0.5).bfloat16()
    h = torch.randn(T, cfg.hidden, device="cuda").bfloat16()
    nxt = w["text/layers/2/input_norm"]
    model.moe = MoeBlock(cfg, "cuda", ws.max_tokens, expert_format="fp8_block")
    for rep in range(2):
        ws.x[:T].copy_(x0)
        ws.normed[:T].copy_(h)
        model.moe.forward(model, ws, T, p, nxt, ws.normed[:T])
        torch.cuda.synchronize()
        model.status.check()
    # oracle
    hf = h.float().cpu()
    router = R.bf16_round(hf @ w[f"{p}/moe/router"].float().cpu().t())
    wts, ids = R.moe_route(router[:, : m.n_experts], m.top_k, True)
    gu = Q.dequant_fp8_block128(*Q.quantize_fp8_block128(w[f"{p}/moe/experts_gate_up"])).cpu()
    dn = Q.dequant_fp8_block128(*Q.quantize_fp8_block128(w[f"{p}/moe/experts_down"])).cpu()
    hq = Q.fake_quant_fp8_block128_rows(hf)
    out = torch.zeros(T, cfg.hidden)
    for t in range(T):
        for j in range(m.top_k):
            e = int(ids[t, j])
            g = hq[t] @ gu[e].t()
            act = R.bf16_round(torch.nn.functional.silu(g[: m.expert_inter]) * g[m.expert_inter:])
            y = R.bf16_round(Q.fake_quant_fp8_block128_rows(act[None])[0] @ dn[e].t())
            out[t] += wts[t, j] * y
    sg = hf @ w[f"{p}/moe/shared_gate_up"].float().cpu().t()
    sact = R.bf16_round(torch.nn.functional.silu(sg[:, : m.shared_inter]) * sg[:, m.shared_inter:])
    shared = R.bf16_round(sact @ w[f"{p}/moe/shared_down"].float().cpu().t())
    want = R.bf16_round(x0.float().cpu() + out + torch.sigmoid(router[:, m.n_experts:]) * shared)
    same = (model.moe.ids[:T].cpu().long() == ids).all(-1)
    assert same.float().mean().item() >= 0.97
    err = (ws.x[:T].float().cpu() - want)[same].abs().max().item()
    assert err <= 0.02 * want.abs().max().item() + 0.02, err
