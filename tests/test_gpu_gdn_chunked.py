"""Chunked (WY) tensor-core gated delta rule against the fp32 token-by-token oracle and the recurrent kernel."""
import pytest
import torch

from ninfer_fusion_b200.ops import reference as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ninfer_fusion_b200._lib import load_native
    return load_native()


@pytest.mark.parametrize("heads", [(2, 6), (16, 48)])
@pytest.mark.parametrize("lens", [[300, 40], [64, 3], [129, 64, 1], [1000]])
def test_gdn_chunked_matches_oracle(ops, lens, heads):
    torch.manual_seed(4)
    (hk, hv), d = heads, 128
    qk, vd = hk * d, hv * d
    C = 2 * qk + vd
    ld = C + vd + 2 * hv
    ld = (ld + 7) // 8 * 8
    T, B = sum(lens), len(lens)
    proj = (torch.randn(T, ld) * 0.7).to(torch.bfloat16)
    conv = (torch.randn(T, C) * 0.8).to(torch.bfloat16)      # stands for the conv + SiLU output
    A_log = torch.rand(hv) * 2 - 1
    dt_bias = torch.rand(hv) * 2 - 1.5
    nw = (1 + 0.1 * torch.randn(d)).to(torch.bfloat16)
    slots = [3, 0, 2][:B]
    n_slots = 4
    ssm = torch.randn(n_slots, hv, d, d) * 0.1
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
    slot_t = torch.tensor(slots).int().cuda()
    args = (conv.cuda(), 0, qk, 2 * qk, proj.cuda(), C, C + vd, C + vd + hv, hk, hv, A_log.cuda(), dt_bias.cuda(),
            nw.cuda(), 1e-6, cu, slot_t)
    ws = torch.empty(int(ops.gdn_chunked_workspace_bytes(T, B, hv)), dtype=torch.uint8, device="cuda")

    ssm_c = ssm.clone().cuda()
    out_c = torch.full((T, vd), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gdn_recurrent(*args, ssm_c, True, out_c, False, None, None, ws)
    ssm_r = ssm.clone().cuda()
    out_r = torch.empty_like(out_c)
    ops.gdn_recurrent(*args, ssm_r, True, out_r, False, None, None, None)
    torch.cuda.synchronize()
    assert not torch.isnan(out_c).any()
    # a verify-style pass leaves the state untouched
    ssm_v = ssm.clone().cuda()
    out_v = torch.empty_like(out_c)
    ops.gdn_recurrent(*args, ssm_v, False, out_v, False, None, None, ws)
    assert torch.equal(ssm_v.cpu(), ssm) and torch.equal(out_v, out_c)

    worst_o = worst_s = 0.0
    for b, n in enumerate(lens):
        s, e = int(cu[b]), int(cu[b + 1])
        pj = proj[s:e].float()
        cref = conv[s:e].float()
        q = cref[:, :qk].view(n, hk, d)
        k = cref[:, qk:2 * qk].view(n, hk, d)
        v = cref[:, 2 * qk:].view(n, hv, d)
        z = pj[:, C:C + vd].view(n, hv, d)
        g, beta = R.gdn_gating(pj[:, C + vd:C + vd + hv], pj[:, C + vd + hv:C + vd + 2 * hv], A_log, dt_bias)
        o, new_s = R.gdn_recurrent(q, k, v, g, beta, ssm[slots[b]])
        y = R.gated_rmsnorm(R.bf16_round(o), z, nw).view(n, vd)
        scale = max(1.0, y.abs().max().item())
        worst_o = max(worst_o, (out_c[s:e].float().cpu() - y).abs().max().item() / scale)
        worst_s = max(worst_s, (ssm_c[slots[b]].cpu() - new_s).abs().max().item() / max(1.0, new_s.abs().max().item()))
    print(f"chunked vs oracle: out {worst_o:.4f} state {worst_s:.5f}; "
          f"vs recurrent kernel: out {(out_c.float() - out_r.float()).abs().max().item():.4f} "
          f"state {(ssm_c - ssm_r).abs().max().item():.5f}")
    assert worst_o < 0.06, worst_o
    assert worst_s < 1e-2, worst_s
    for s_ in [s for s in range(n_slots) if s not in slots]:
        assert torch.equal(ssm_c[s_].cpu(), ssm[s_])
