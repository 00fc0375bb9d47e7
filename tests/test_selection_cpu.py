"""Block selector + selected-block attention oracle: a small selection reproduces full attention when the mass is
concentrated, and the selection always holds the sink and the recent blocks."""
import torch

from ninfer_fusion_b200.ops import reference as R
from ninfer_fusion_b200.ops import selection as S


def test_selector_keeps_sink_recent_and_the_relevant_blocks():
    g = torch.Generator().manual_seed(0)
    Hq, Hkv, D, n = 8, 2, 64, 1003
    k = torch.randn((n, Hkv, D), generator=g) * 0.3
    v = torch.randn((n, Hkv, D), generator=g)
    q = torch.randn((Hq, D), generator=g)
    hot = [37, 120, 201]                                        # blocks whose keys line up with the queries
    for b in hot:
        for h in range(Hkv):
            k[4 * b:4 * b + 4, h] = q[h * 4] * 1.5 + torch.randn((4, D), generator=g) * 0.05
    summ = S.block_summaries(k)
    assert summ.shape == (250, Hkv, D)
    ids, count = S.select_blocks(q, summ, kv_len=n, budget=24, recent=4, sink=1, max_blocks=64)
    chosen = set(ids[:count].tolist())
    assert count == 24 and ids.dtype == torch.int32 and ids[:count].tolist() == sorted(chosen)
    assert 0 in chosen and {246, 247, 248, 249} <= chosen and set(hot) <= chosen
    assert max(chosen) < n // 4
    # attention over the selection (+ the 3 tail tokens) is close to full attention: the mass sits in the hot blocks
    kv_len = torch.tensor([n])
    vis = R.selected_block_mask(kv_len, ids[None], torch.tensor([count]), n)
    full = R.gqa_attention(q[None], k, v, kv_len, 1 / 8)
    sparse = R.gqa_attention(q[None], k, v, None, 1 / 8, vis)
    heads = [0, 4]                                              # the heads the hot blocks were built for
    err = (full - sparse)[0, heads].abs().max() / full[0, heads].abs().max()
    assert err < 0.05
    # a budget smaller than sink + recent still keeps them; a short history selects everything it has
    ids2, c2 = S.select_blocks(q, summ, kv_len=n, budget=2, recent=4, sink=1, max_blocks=64)
    assert c2 == 5
    ids3, c3 = S.select_blocks(q, summ, kv_len=13, budget=24, max_blocks=64)
    assert c3 == 3 and ids3[:3].tolist() == [0, 1, 2]
    assert S.select_blocks(q, summ, kv_len=3, budget=8)[1] == 0
