"""CPU tests of the fp32 oracles and the host-side step plumbing."""
import math

import torch

from ninfer_fusion_b200.kv import codec_report
from ninfer_fusion_b200.models.config import QWEN36_27B, QWEN36_35B_A3B, TINY_DENSE, TINY_MOE
from ninfer_fusion_b200.models.hybrid import pick_attention_split
from ninfer_fusion_b200.models.reference_model import ReferenceModel, ReferenceSequence
from ninfer_fusion_b200.models.weights import random_weights, weight_shapes
from ninfer_fusion_b200.ops import reference as R
from ninfer_fusion_b200.runtime.batch import SeqChunk, StepBuffers
from ninfer_fusion_b200.runtime.kv_cache import GdnStatePool, PagedKvCache


def test_config_geometry():
    c = QWEN36_27B
    assert c.attn_in_dim == 14336 and c.gdn_conv_dim == 10240 and c.gdn_in_dim == 16384 + 96
    assert len(c.attn_layers) == 16 and c.attn_layers[0] == 3
    assert abs(c.param_count() / 1e9 - 26.9) < 0.2
    assert abs(QWEN36_35B_A3B.param_count() / 1e9 - 34.7) < 0.3
    names = [n for n, _, _ in weight_shapes(TINY_MOE, with_mtp=True)]
    assert "mtp/fc" in names and "text/layers/0/moe/router" in names and len(set(names)) == len(names)


def test_codecs_are_idempotent_and_ordered():
    torch.manual_seed(0)
    x = torch.randn(64, 2, 256)
    errs = {}
    for name, fmt, g in [("bf16", R.KV_BF16, 256), ("fp8", R.KV_FP8_ROW, 256), ("int8", R.KV_INT8_GROUP, 64),
                         ("nvfp4", R.KV_NVFP4, 16)]:
        y = R.kv_quant_dequant(x, fmt, g)
        assert torch.equal(R.kv_quant_dequant(y, fmt, g), y) or fmt == R.KV_INT8_GROUP or fmt == R.KV_NVFP4
        errs[name] = (y - R.bf16_round(x)).abs().mean().item()
    assert errs["bf16"] == 0 and errs["int8"] < errs["fp8"] < errs["nvfp4"]


def test_e2m1_rounding_ties_to_even():
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.3, 0.24])
    assert R.e2m1_round(x).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.5, 0.0]


def test_codec_report_config():
    rep = codec_report.run()
    c = rep["codecs"]
    assert c["bf16"]["max_abs_err"] == 0
    assert c["bf16"]["bytes_per_token"] == 2 * 2 * 128 * 2
    assert c["fp8-e4m3-row"]["bytes_per_token"] == 2 * 2 * (128 + 2)
    assert c["int8-g32"]["bytes_per_token"] == 2 * 2 * (128 + 2 * 4)
    assert c["int8-g32"]["mean_abs_err"] < c["fp8-e4m3-row"]["mean_abs_err"] < c["nvfp4-g16"]["mean_abs_err"] < 0.2
    # the K row scale helps nvfp4 on keys with loud channels; the lattice tier needs the rotated frame for them
    assert c["nvfp4-g16+rowscale"]["mean_abs_err"] < 0.9 * c["nvfp4-g16"]["mean_abs_err"]
    assert c["e8-rk4v4+hadamard"]["mean_abs_err"] < 0.6 * c["e8-rk4v4"]["mean_abs_err"]
    assert c["e8-rk4v4"]["bytes_per_token"] < c["nvfp4-g16"]["bytes_per_token"]


def test_gdn_chunk_invariance():
    """Recurrence split at any point gives the same outputs and state."""
    torch.manual_seed(1)
    T, hk, hv, d = 9, 1, 2, 128
    q, k, v = torch.randn(T, hk, d), torch.randn(T, hk, d), torch.randn(T, hv, d)
    g, beta = -torch.rand(T, hv), torch.rand(T, hv)
    s0 = torch.randn(hv, d, d) * 0.1
    o, s = R.gdn_recurrent(q, k, v, g, beta, s0)
    o1, s1 = R.gdn_recurrent(q[:4], k[:4], v[:4], g[:4], beta[:4], s0)
    o2, s2 = R.gdn_recurrent(q[4:], k[4:], v[4:], g[4:], beta[4:], s1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-5) and torch.allclose(s2, s, atol=1e-5)


def test_reference_model_prefill_equals_stepwise():
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=3, std=0.05)
    m = ReferenceModel(cfg, w)
    ids = torch.randint(0, cfg.vocab, (11,))
    a = m.forward(ReferenceSequence(cfg), ids)
    seq = ReferenceSequence(cfg)
    b = torch.cat([m.forward(seq, ids[i:i + 1]) for i in range(11)])
    assert (a - b).abs().max().item() < 0.08  # bf16 rounding points differ only through summation order


def test_moe_reference_runs_and_routes():
    cfg = TINY_MOE
    w = random_weights(cfg, "cpu", seed=4, std=0.05)
    m = ReferenceModel(cfg, w)
    out = m.generate_greedy(torch.randint(0, cfg.vocab, (6,)), 3)
    assert len(out) == 3
    wts, ids = R.moe_route(torch.tensor([[1.0, 3.0, 3.0, 0.0]]), 2)
    assert ids.tolist() == [[1, 2]] and abs(wts.sum().item() - 1) < 1e-6


def test_step_buffers_and_paging():
    sb = StepBuffers(64, 4, "cpu")
    b = sb.build([SeqChunk(0, 1, 5, [1, 2, 3]), SeqChunk(2, 0, 0, [9], True)])
    assert b.ids.tolist() == [1, 2, 3, 9] and b.cache_pos.tolist() == [5, 6, 7, 0]
    assert b.kv_len.tolist() == [6, 7, 8, 1] and b.cu_seqlens.tolist() == [0, 3, 4]
    assert b.logit_rows.tolist() == [2, 3] and b.table_row.tolist() == [0, 0, 0, 2] and b.max_kv_len == 8
    kv = PagedKvCache(TINY_DENSE, 10, 16, 4, 8, "cpu", formats="fp8")
    kv.ensure(0, 17)
    kv.ensure(1, 1)
    assert kv.pool.free_pages == 7 and (kv.table_host[0, :2] >= 0).all() and kv.table_host[0, 2] == -1
    kv.fork_row(0, 2, 17)  # one shared full page + a copied partial tail
    assert kv.pool.free_pages == 6 and kv.table_host[2, 0] == kv.table_host[0, 0] and kv.table_host[2, 1] != kv.table_host[0, 1]
    kv.trim(0, 16)
    kv.free_row(0)
    kv.free_row(2)
    kv.free_row(1)
    assert kv.pool.free_pages == 10
    assert abs(kv.bytes_per_token() - 1 * 2 * 1 * (256 + 2)) < 1e-6
    st = GdnStatePool(TINY_DENSE, 3, "cpu")
    s = st.alloc()
    st.ssm[0][s].fill_(1.0)
    t = st.alloc()
    st.copy_slot(s, t)
    assert st.ssm[0][t].sum().item() == st.ssm[0][s].numel()


def test_attention_split_geometry_is_bucketed():
    a = pick_attention_split(2049, 128)
    b = pick_attention_split(4000, 128)
    assert a[0] == b[0] and a[0] % 128 == 0          # same bucket -> same absolute key ranges
    assert pick_attention_split(2048, 100000)[1] == 1  # prefill: plenty of parallelism, no split
    s, n = pick_attention_split(131072, 8, max_splits=64)
    assert n <= 64 and s * n >= 131072
