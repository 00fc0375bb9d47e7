"""Mixed-precision KV layers: cells of one layer in three tiers (bf16 / fp8-row / nvfp4), attention and append
following the cell map, the re-encoding kernel, and the engine-driven descent that frees device bytes."""
import pytest
import torch

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.ops import reference as R
from ninfer_fusion_b200.runtime.kv_cache import PagedKvCache

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ninfer_fusion_b200._lib import load_native
    return load_native()


def _oracle_rows(x_bf16, tier):
    """What a cell holds after descending to `tier` one rung at a time."""
    y = x_bf16
    if tier >= 1:
        y = R.kv_quant_dequant(y, R.KV_FP8_ROW, 256)
    if tier >= 2:
        y = R.kv_quant_dequant(y, R.KV_NVFP4, 16, bf16_input=False)   # the device re-encodes the fp32 decode
    return y


def test_attention_over_pages_at_three_rungs_matches_per_page_oracle(ops):
    torch.manual_seed(3)
    cfg = TINY_DENSE
    hq, hkv, D, P = 6, 1, 256, 64
    n = 333                                    # six pages, the last one partial
    kv = PagedKvCache(cfg, 12, P, 2, 8, "cuda", formats="mixed", n_kv_heads=hkv, n_layers=1, mixed_capacity=(8, 8, 8))
    L = kv.layers[0]
    kv.ensure(0, n + 1)
    kv.publish()
    inv_freq = R.rope_inv_freq(64, 1e7).cuda()
    ld = (2 * hq + 2 * hkv) * D
    proj = torch.randn(n, ld).to(torch.bfloat16).cuda()
    tok_seq = torch.zeros(n, dtype=torch.int32, device="cuda")
    pos = torch.arange(n).int().cuda()
    q = torch.empty((n, hq, D), dtype=torch.bfloat16, device="cuda")
    k_off, v_off = hq * D, hq * D + hkv * D + hq * D

    def prep(rows):
        ops.attn_prep(proj[rows], 0, k_off, v_off, hq, hkv, D, None, None, 1e-6, True, 0, inv_freq, 1.0, pos[rows],
                      tok_seq[rows], pos[rows], kv.table, q[rows], L.k_codes, L.v_codes, None, None, P, L.fmt, L.group,
                      False, False, None, L.desc)

    first = slice(0, 300)
    prep(first)                                # 300 tokens appended at the hot tier (bf16)
    pages = kv.row_pages[0]
    assert kv.tier_census() == {"bf16": 6, "fp8": 0, "nvfp4": 0}
    bytes_hot = kv.bytes_in_use()
    assert kv.descend(0, pages[:4], 1) == 4    # pages 0..3 -> fp8
    assert kv.descend(0, pages[:2], 2) == 2    # pages 0..1 -> nvfp4 (from their fp8 contents)
    assert kv.descend(0, pages[:2], 2) == 0    # already there
    assert kv.tier_census() == {"bf16": 2, "fp8": 2, "nvfp4": 2}
    assert kv.bytes_in_use() < bytes_hot
    prep(slice(300, n))                        # later tokens keep arriving in the hot tier
    tier_of_page = [2, 2, 1, 1, 0, 0]

    pf = proj.float().cpu()
    k_all = R.bf16_round(pf[:, k_off:k_off + hkv * D].view(n, hkv, D))
    v_all = R.bf16_round(pf[:, v_off:v_off + hkv * D].view(n, hkv, D))
    k_ref, v_ref = k_all.clone(), v_all.clone()
    for pg, t in enumerate(tier_of_page):
        lo, hi = pg * P, min(n, (pg + 1) * P)
        rows = slice(lo, min(hi, 300)) if t else slice(lo, hi)   # only what was there when the cell descended
        k_ref[rows] = _oracle_rows(k_all[rows], t)
        v_ref[rows] = _oracle_rows(v_all[rows], t)
    i = torch.arange(n)
    causal = i[None, :] <= i[:, None]
    ref = R.bf16_round(R.gqa_attention(q.float().cpu(), k_ref, v_ref, None, 1 / 16, causal)).reshape(n, -1)

    # decode-shaped queries through the split-KV tensor-core kernel
    rows = torch.tensor([n - 1, 299, 130, 64]).cuda()
    qd = q[rows].contiguous()
    kv_len = (pos + 1).contiguous()
    for split_keys, n_splits in ((128, 3), (512, 1)):
        od = torch.full((len(rows), hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        part_o = torch.empty(len(rows) * hq * n_splits * D, device="cuda")
        part_ml = torch.empty(len(rows) * hq * n_splits * 2, device="cuda")
        ops.paged_attention(qd, hq, hkv, D, tok_seq[rows].contiguous(), kv_len[rows].contiguous(), kv.table, L.k_codes,
                            L.v_codes, None, None, P, L.fmt, L.group, 1 / 16, split_keys, n_splits, part_o, part_ml, None,
                            od, None, None, 2, False, 0, None, None, L.desc)
        err = (od.float().cpu() - ref[rows.cpu()]).abs().max().item()
        assert err < 0.04, f"split {split_keys}: {err}"

    # the prefill kernel over the whole sequence
    qt = int(ops.prefill_attn_block_tokens(hq, hkv))
    blk_s = list(range(0, n, qt))
    blk_c = [min(qt, n - s) for s in blk_s]
    out = torch.full((n, hq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.paged_attention_prefill(q, hq, hkv, D, tok_seq, kv_len, torch.tensor(blk_s).int().cuda(),
                                torch.tensor(blk_c).int().cuda(), kv.table, L.k_codes, L.v_codes, None, None, P, L.fmt,
                                L.group, 1 / 16, None, out, False, 0, L.desc)
    assert not torch.isnan(out).any()
    assert (out.float().cpu() - ref).abs().max().item() < 0.04

    # freeing the row gives every cell back, whatever tier it ended in
    kv.free_row(0)
    assert kv.tier_census() == {"bf16": 0, "fp8": 0, "nvfp4": 0} and kv.pool.free_pages == 12


def test_engine_descent_frees_kv_bytes_and_keeps_generating():
    """An engine whose program descends cells older than 128 tokens down to a byte target: resident KV bytes fall
    to the target while the request keeps decoding, and the tokens stay close to the run without descent."""
    from ninfer_fusion_b200.kv.descent import DescentConfig
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.engine import Engine, RequestOptions
    from ninfer_fusion_b200.runtime.gpu_program import GpuProgram

    cfg = TINY_DENSE
    w = random_weights(cfg, "cuda", seed=4, std=0.05)
    torch.manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (700,)).tolist()
    n_new = 40

    def run(descent):
        import time

        def factory():
            return GpuProgram(cfg, w, "cuda", max_lanes=2, max_context=1024, kv_format="mixed", page_size=64,
                              prefill_chunk=256, mixed_capacity=(16, 16, 16), descent=descent)
        eng = Engine(factory, prefill_chunk=256)
        try:
            h = eng.submit(prompt, RequestOptions(max_tokens=n_new))
            seen = []     # (bytes in use, cells per tier) while the lane is alive
            while h.t_done is None:
                c = eng.health().get("census", {})
                if c.get("kv_bytes_in_use"):
                    seen.append((c["kv_bytes_in_use"], c["kv_tiers"]))
                time.sleep(0.002)
            toks = h.wait(timeout=300)
            return toks, seen, dict(eng.program.descent_stats)
        finally:
            eng.shutdown()

    base, seen0, stats0 = run(None)
    assert len(base) == n_new and stats0["cells_moved"] == 0
    # one full-attention layer in the tiny model, 12 pages of 64 tokens at the end of the run: a bf16 cell is 64 KiB
    hot_cell = 2 * 64 * 256 * 2
    assert max(b for b, _ in seen0) >= 11 * hot_cell
    target = 6 * hot_cell
    cfg_d = DescentConfig(min_age_tokens=128, max_cells_per_pass=4, target_resident_bytes=target, sink_blocks=1)
    toks, seen, stats = run(cfg_d)
    assert len(toks) == n_new and stats["cells_moved"] > 0
    assert seen and seen[-1][0] <= 1.1 * target, f"resident KV bytes {seen[-1]} did not fall to the target {target}"
    assert seen[-1][1]["fp8"] + seen[-1][1]["nvfp4"] > 0
    same = sum(int(a == b) for a, b in zip(base, toks))
    assert same >= n_new // 2, f"only {same} of {n_new} tokens agree with the run without descent"
