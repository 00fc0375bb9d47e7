"""tcgen05 split-KV decode attention over fp8-row pages (csrc/attention/paged_attention_tc.cu) against the fp32
oracle that dequantises the same pages: GQA groups of 3 / 6 / 8 / 16 rows, pages of 64 and 128 tokens, scattered page
tables, several split sizes, a sliding window, tree-verify masks, rows with very different V scales, and the
equality of the partial-result contract with the mma.sync kernel (the merge kernel is shared)."""
import math

import pytest
import torch

from ninfer_fusion_b200.ops import reference as R

pytestmark = pytest.mark.gpu
D = 256


@pytest.fixture(scope="module")
def ops():
    from ninfer_fusion_b200._lib import load_native
    return load_native()


def _fill(ops, lens, hq, hkv, P, v_row_gain=None, seed=1):
    """Appends random K / V for sequences of `lens` tokens into scattered fp8-row pages through attn_prep."""
    torch.manual_seed(seed)
    B = len(lens)
    max_pages = (max(lens) + P - 1) // P
    n_pages = B * max_pages + 3
    table = torch.randperm(n_pages)[: B * max_pages].int().view(B, max_pages).cuda()
    k_codes = torch.zeros((n_pages, hkv, P, D), dtype=torch.uint8, device="cuda")
    v_codes = torch.zeros_like(k_codes)
    k_sc = torch.zeros((n_pages, hkv, P, 2), dtype=torch.uint8, device="cuda")
    v_sc = torch.zeros_like(k_sc)
    T = sum(lens)
    ld = (2 * hq + 2 * hkv) * D
    proj = torch.randn(T, ld)
    k_off, v_off = hq * D, hq * D + hkv * D + hq * D
    for c in torch.randperm(D)[:4]:
        proj[:, k_off + c] *= 8                       # K outlier channels
    if v_row_gain is not None:
        proj[:, v_off:v_off + hkv * D] *= v_row_gain.view(T, 1)
    proj = proj.to(torch.bfloat16).cuda()
    tok_seq = torch.cat([torch.full((n,), b) for b, n in enumerate(lens)]).int().cuda()
    pos = torch.cat([torch.arange(n) for n in lens]).int().cuda()
    q = torch.empty((T, hq, D), dtype=torch.bfloat16, device="cuda")
    inv_freq = R.rope_inv_freq(64, 1e7).cuda()
    ops.attn_prep(proj, 0, k_off, v_off, hq, hkv, D, None, None, 1e-6, True, 0, inv_freq, 1.0, pos, tok_seq, pos, table,
                  q, k_codes, v_codes, k_sc, v_sc, P, R.KV_FP8_ROW, D, False)
    pf = proj.float().cpu()
    k_ref = R.kv_quant_dequant(pf[:, k_off:k_off + hkv * D].view(T, hkv, D), R.KV_FP8_ROW, D)
    v_ref = R.kv_quant_dequant(pf[:, v_off:v_off + hkv * D].view(T, hkv, D), R.KV_FP8_ROW, D)
    return dict(q=q, table=table, planes=(k_codes, v_codes, k_sc, v_sc), k_ref=k_ref, v_ref=v_ref, T=T)


def _attend(ops, f, hq, hkv, P, rows, seqs, kv_lens, split_keys, impl, window=0, masks=None, base=None, max_len=None):
    q = f["q"][torch.tensor(rows).cuda()].contiguous()
    Tq = len(rows)
    n_splits = ((max_len or max(kv_lens)) + split_keys - 1) // split_keys
    part_o = torch.full((Tq * hq * n_splits * D,), float("nan"), device="cuda")
    part_ml = torch.full((Tq * hq * n_splits * 2,), float("nan"), device="cuda")
    out = torch.full((Tq, hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
    k_codes, v_codes, k_sc, v_sc = f["planes"]
    ops.paged_attention(q, hq, hkv, D, torch.tensor(seqs).int().cuda(), torch.tensor(kv_lens).int().cuda(), f["table"],
                        k_codes, v_codes, k_sc, v_sc, P, R.KV_FP8_ROW, D, 1 / math.sqrt(D), split_keys, n_splits,
                        part_o, part_ml, None, out, masks, base, impl, False, window)
    torch.cuda.synchronize()
    return out.float().cpu(), q.float().cpu()


@pytest.mark.parametrize("hq,hkv,P", [(24, 4, 64), (6, 1, 64), (3, 1, 64), (16, 2, 128), (16, 1, 64)])
@pytest.mark.parametrize("split_keys", [128, 256, 512])
def test_matches_the_oracle_over_scattered_fp8_pages(ops, hq, hkv, P, split_keys):
    lens = [37, 256, 1000, 300, 129]
    f = _fill(ops, lens, hq, hkv, P)
    rows, seqs, kv_lens, start = [], [], [], 0
    starts = [0]
    for b, n in enumerate(lens):
        for p in sorted({n - 1, n // 2, min(n - 1, 127), min(n - 1, 128)}):
            rows.append(start + p); seqs.append(b); kv_lens.append(p + 1)
        start += n
        starts.append(start)
    out, q = _attend(ops, f, hq, hkv, P, rows, seqs, kv_lens, split_keys, 3)
    for i in range(len(rows)):
        b = seqs[i]
        ref = R.gqa_attention(q[i:i + 1], f["k_ref"][starts[b]:starts[b + 1]], f["v_ref"][starts[b]:starts[b + 1]],
                              torch.tensor([kv_lens[i]]))
        err = (out[i] - R.bf16_round(ref).view(-1)).abs().max().item()
        assert err < 0.03, f"query {i} (kv_len {kv_lens[i]}): err {err}"


def test_agrees_with_the_mma_sync_kernel_and_handles_v_scales_six_orders_apart(ops):
    hq, hkv, P = 6, 1, 64
    lens = [700]
    gain = torch.ones(700)
    gain[::7] = 1e-3                                   # rows whose V scale is far below the running maximum
    gain[350] = 1e3                                    # and one far above everything before it
    f = _fill(ops, lens, hq, hkv, P, v_row_gain=gain, seed=5)
    rows, seqs = [699, 349, 351], [0, 0, 0]
    kv_lens = [r + 1 for r in rows]
    a, q = _attend(ops, f, hq, hkv, P, rows, seqs, kv_lens, 256, 3)
    b, _ = _attend(ops, f, hq, hkv, P, rows, seqs, kv_lens, 256, 2)
    for i in range(3):
        ref = R.bf16_round(R.gqa_attention(q[i:i + 1], f["k_ref"], f["v_ref"], torch.tensor([kv_lens[i]]))).view(-1)
        scale = ref.abs().max().item()
        assert (a[i] - ref).abs().max().item() < 0.02 * max(1.0, scale), f"tcgen05 query {i}"
        assert (a[i] - b[i]).abs().max().item() < 0.02 * max(1.0, scale), f"kernels disagree on query {i}"


def test_sliding_window_and_tree_masks(ops):
    hq, hkv, P = 6, 1, 64
    L, W = 330, 5
    f = _fill(ops, [L + W], hq, hkv, P, seed=7)
    # window: the last 200 keys only
    out, q = _attend(ops, f, hq, hkv, P, [L - 1], [0], [L], 128, 3, window=200)
    vis = torch.zeros(1, L + W, dtype=torch.bool)
    vis[0, L - 200:L] = True
    ref = R.bf16_round(R.gqa_attention(q, f["k_ref"], f["v_ref"], None, 1 / 16, vis)).view(-1)
    assert (out[0] - ref).abs().max().item() < 0.03
    # tree: node j sees the prefix and its ancestors among the W appended nodes
    anc = [[0], [0, 1], [0, 2], [0, 1, 3], [0, 2, 4]]
    masks = torch.tensor([sum(1 << a for a in row) for row in anc], dtype=torch.long).cuda()
    base = torch.full((W,), L, dtype=torch.int32).cuda()
    rows = [L + j for j in range(W)]
    out, q = _attend(ops, f, hq, hkv, P, rows, [0] * W, [L + W] * W, 256, 3, masks=masks, base=base)
    vis = torch.zeros(W, L + W, dtype=torch.bool)
    vis[:, :L] = True
    for j, row in enumerate(anc):
        for a in row:
            vis[j, L + a] = True
    ref = R.bf16_round(R.gqa_attention(q, f["k_ref"], f["v_ref"], None, 1 / 16, vis)).reshape(W, -1)
    assert (out - ref).abs().max().item() < 0.03


def test_more_items_than_sms_and_released_pages(ops):
    """A batch large enough that every persistent CTA walks several items; one sequence has a released page (-1)
    whose keys must contribute nothing."""
    hq, hkv, P = 8, 2, 64
    lens = [520] * 24
    f = _fill(ops, lens, hq, hkv, P, seed=9)
    f["table"][3, 2] = -1                               # keys 128..191 of sequence 3 are gone
    rows = [b * 520 + 519 for b in range(24)]
    out, q = _attend(ops, f, hq, hkv, P, rows, list(range(24)), [520] * 24, 128, 3)
    for b in (0, 3, 23):
        k, v = f["k_ref"][b * 520:(b + 1) * 520], f["v_ref"][b * 520:(b + 1) * 520]
        vis = torch.ones(1, 520, dtype=torch.bool)
        if b == 3:
            vis[0, 128:192] = False
        ref = R.bf16_round(R.gqa_attention(q[b:b + 1], k, v, None, 1 / 16, vis)).view(-1)
        assert (out[b] - ref).abs().max().item() < 0.03, f"sequence {b}"
