"""Sliding-window attention: prefill blocks and both split-KV decode kernels against the fp32 oracle with a window mask."""
import pytest
import torch

from ninfer_fusion_b200.ops import reference as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ninfer_fusion_b200._lib import load_native
    return load_native()


@pytest.mark.parametrize("window", [1, 48, 100, 4096])
def test_window_prefill_and_decode(ops, window):
    torch.manual_seed(11)
    hq, hkv, D, P = 6, 1, 256, 16
    fmt, group = R.KV_BF16, D
    lens = [333, 70]
    B = len(lens)
    max_pages = (max(lens) + P - 1) // P
    n_pages = B * max_pages + 2
    table = torch.randperm(n_pages)[: B * max_pages].int().view(B, max_pages).cuda()
    k_codes = torch.zeros((n_pages, hkv, P, 2 * D), dtype=torch.uint8, device="cuda")
    v_codes = torch.zeros_like(k_codes)
    inv_freq = R.rope_inv_freq(64, 1e7).cuda()
    ld = (2 * hq + 2 * hkv) * D
    T = sum(lens)
    proj = torch.randn(T, ld).to(torch.bfloat16).cuda()
    tok_seq = torch.cat([torch.full((n,), b) for b, n in enumerate(lens)]).int().cuda()
    pos = torch.cat([torch.arange(n) for n in lens]).int().cuda()
    q = torch.empty((T, hq, D), dtype=torch.bfloat16, device="cuda")
    k_off, v_off = hq * D, hq * D + hkv * D + hq * D
    ops.attn_prep(proj, 0, k_off, v_off, hq, hkv, D, None, None, 1e-6, True, 0, inv_freq, 1.0, pos, tok_seq, pos, table,
                  q, k_codes, v_codes, None, None, P, fmt, group, False)
    kv_len = (pos + 1).contiguous()
    qt = int(ops.prefill_attn_block_tokens(hq, hkv))
    blk_s, blk_c, t = [], [], 0
    for n in lens:
        for o in range(0, n, qt):
            blk_s.append(t + o)
            blk_c.append(min(qt, n - o))
        t += n
    out = torch.full((T, hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.paged_attention_prefill(q, hq, hkv, D, tok_seq, kv_len, torch.tensor(blk_s).int().cuda(),
                                torch.tensor(blk_c).int().cuda(), table, k_codes, v_codes, None, None, P, fmt, group,
                                1 / 16, None, out, False, window)
    pf = proj.float().cpu()
    k_all = R.bf16_round(pf[:, k_off:k_off + hkv * D].view(T, hkv, D))
    v_all = R.bf16_round(pf[:, v_off:v_off + hkv * D].view(T, hkv, D))
    starts = [0, lens[0]]
    ref = torch.empty(T, hq * D)
    for b, n in enumerate(lens):
        s = starts[b]
        i = torch.arange(n)
        vis = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - window)
        o = R.gqa_attention(q[s:s + n].float().cpu(), k_all[s:s + n], v_all[s:s + n], None, 1 / 16, vis)
        ref[s:s + n] = R.bf16_round(o).reshape(n, -1)
    assert not torch.isnan(out).any()
    assert (out.float().cpu() - ref).abs().max().item() < 0.03

    # decode-shaped queries: the last token of each sequence plus two mid-sequence ones, both kernels, two split sizes
    rows = torch.tensor([lens[0] - 1, T - 1, 200, lens[0] + 5]).cuda()
    qd = q[rows].contiguous()
    for impl in (1, 2):
        for split_keys, n_splits in ((128, 3), (512, 1)):
            od = torch.full((len(rows), hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
            part_o = torch.empty(len(rows) * hq * n_splits * D, device="cuda")
            part_ml = torch.empty(len(rows) * hq * n_splits * 2, device="cuda")
            ops.paged_attention(qd, hq, hkv, D, tok_seq[rows].contiguous(), kv_len[rows].contiguous(), table, k_codes,
                                v_codes, None, None, P, fmt, group, 1 / 16, split_keys, n_splits, part_o, part_ml, None,
                                od, None, None, impl, False, window)
            err = (od.float().cpu() - ref[rows.cpu()]).abs().max().item()
            assert err < 0.03, f"impl {impl} split {split_keys}: {err}"


@pytest.mark.parametrize("window", [48, 100])
def test_window_decode_with_released_pages_fp8(ops, window):
    """A windowed row whose early pages went back to the pool (block-table entries -1, the convention of
    PagedKvCache.release_before): the split-KV kernels and the prefill kernel must neither read those pages'
    codes nor their row scales, and the result equals the windowed oracle on the fp8-row codec."""
    torch.manual_seed(5)
    hq, hkv, D, P = 6, 1, 256, 16
    fmt, group = R.KV_FP8_ROW, D
    n = 333
    max_pages = (n + P - 1) // P
    n_pages = max_pages + 2
    table = torch.randperm(n_pages)[:max_pages].int().view(1, max_pages).cuda()
    k_codes = torch.zeros((n_pages, hkv, P, D), dtype=torch.uint8, device="cuda")
    v_codes = torch.zeros_like(k_codes)
    k_sc = torch.zeros((n_pages, hkv, P, 2), dtype=torch.uint8, device="cuda")
    v_sc = torch.zeros_like(k_sc)
    inv_freq = R.rope_inv_freq(64, 1e7).cuda()
    ld = (2 * hq + 2 * hkv) * D
    proj = torch.randn(n, ld).to(torch.bfloat16).cuda()
    tok_seq = torch.zeros(n, dtype=torch.int32, device="cuda")
    pos = torch.arange(n).int().cuda()
    q = torch.empty((n, hq, D), dtype=torch.bfloat16, device="cuda")
    k_off, v_off = hq * D, hq * D + hkv * D + hq * D
    ops.attn_prep(proj, 0, k_off, v_off, hq, hkv, D, None, None, 1e-6, True, 0, inv_freq, 1.0, pos, tok_seq, pos, table,
                  q, k_codes, v_codes, k_sc, v_sc, P, fmt, group, False)
    # oracle on the codec's represented values, before anything is released
    pf = proj.float().cpu()
    k_all = R.kv_quant_dequant(R.bf16_round(pf[:, k_off:k_off + hkv * D].view(n, hkv, D)), fmt, group)
    v_all = R.kv_quant_dequant(R.bf16_round(pf[:, v_off:v_off + hkv * D].view(n, hkv, D)), fmt, group)
    i = torch.arange(n)
    vis = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - window)
    ref = R.bf16_round(R.gqa_attention(q.float().cpu(), k_all, v_all, None, 1 / 16, vis)).reshape(n, -1)[n - 1:n]
    # release what release_before would: pages wholly before n + 1 - window - 64
    first_needed = max(0, n + 1 - window - 64)
    released = first_needed // P
    assert released > 0
    table[0, :released] = -1
    kv_len = torch.tensor([n], dtype=torch.int32, device="cuda")
    qd = q[n - 1:n].contiguous()
    outs = []
    for impl in (1, 2):
        for split_keys, n_splits in ((128, 3), (512, 1)):
            od = torch.full((1, hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
            part_o = torch.empty(hq * n_splits * D, device="cuda")
            part_ml = torch.empty(hq * n_splits * 2, device="cuda")
            ops.paged_attention(qd, hq, hkv, D, tok_seq[:1].contiguous(), kv_len, table, k_codes, v_codes, k_sc, v_sc, P,
                                fmt, group, 1 / 16, split_keys, n_splits, part_o, part_ml, None, od, None, None, impl,
                                False, window)
            assert not torch.isnan(od).any()
            outs.append(od.float().cpu())
    # same query with every page still mapped: released pages lie outside the window, so nothing may change
    table_full = table.clone()
    spare = [p_ for p_ in range(n_pages) if p_ not in set(table[0, released:].tolist())]
    table_full[0, :released] = torch.tensor(spare[:released], dtype=torch.int32)   # any valid page: it is masked anyway
    od = torch.empty((1, hq * D), dtype=torch.bfloat16, device="cuda")
    part_o = torch.empty(hq * 3 * D, device="cuda")
    part_ml = torch.empty(hq * 3 * 2, device="cuda")
    ops.paged_attention(qd, hq, hkv, D, tok_seq[:1].contiguous(), kv_len, table_full, k_codes, v_codes, k_sc, v_sc, P,
                        fmt, group, 1 / 16, 128, 3, part_o, part_ml, None, od, None, None, 2, False, window)
    for o in outs:
        assert (o - od.float().cpu()).abs().max().item() < 0.02
        assert (o - ref).abs().max().item() < 0.04
    # prefill kernel over the last query block of the row
    qt = int(ops.prefill_attn_block_tokens(hq, hkv))
    s0 = (n - 1) // qt * qt
    out = torch.full((n, hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.paged_attention_prefill(q, hq, hkv, D, tok_seq, (pos + 1).contiguous(), torch.tensor([s0]).int().cuda(),
                                torch.tensor([n - s0]).int().cuda(), table, k_codes, v_codes, k_sc, v_sc, P, fmt, group,
                                1 / 16, None, out, False, window)
    assert not torch.isnan(out[s0:]).any()
    assert (out[n - 1:n].float().cpu() - od.float().cpu()).abs().max().item() < 0.03
