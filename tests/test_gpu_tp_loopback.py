"""Tensor-parallel peer-memory kernels, walked through on ONE GPU.

All ranks live in one process, each with its own symmetric allocation
(`TensorParallel.loopback`).  Every collective is launched phase by phase --
first every rank's producing step, then every rank's consuming step -- so every
counter a kernel looks at is already satisfied and no launch ever waits for a
later one.  What is checked: the addressing of the pushes, the counter
arithmetic over several calls in a row, and the numerics against an fp32 sum of
the per-rank products (+ residual, + RMS norm).  The reference tests its rank
logic on one GPU the same way (src/core/virtual_device.h:137-145).
"""
from types import SimpleNamespace

import pytest
import torch

from ninfer_fusion_b200._lib import StatusWord
from ninfer_fusion_b200.models.config import ModelConfig
from ninfer_fusion_b200.parallel.tp import TensorParallel

pytestmark = pytest.mark.gpu

CFG = ModelConfig(name="tp-loopback", n_layers=4, hidden=1024, vocab=2048, n_q_heads=8, n_kv_heads=2, head_dim=256,
                  rot_dim=64, rope_theta=1e7, gdn_qk_heads=8, gdn_v_heads=8, ffn_inter=1024, max_context=4096)
EPS = CFG.rms_eps
EPI_STORE, EPI_SWIGLU = 0, 2


def _models(ops, ranks):
    return [SimpleNamespace(ops=ops, status=StatusWord("cuda"), pdl=False, _gathered=None) for _ in ranks]


def _ws(tp):
    return SimpleNamespace(x=tp.x)


def _rms(x):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + EPS)


def _close(got, want, tol=2e-2):
    scale = want.abs().max().item() + 1e-6
    err = (got.float() - want).abs().max().item()
    assert err <= tol * scale, f"max abs error {err:.4g} against a range of {scale:.4g}"


@pytest.mark.parametrize("world,T,K", [(1, 32, 2048), (1, 7, 512), (2, 32, 512), (2, 1, 768), (4, 100, 256), (8, 32, 128)])
def test_rs_ag_gemm_then_gathered_gemm(ops, world, T, K):
    """GEMM -> reduce-scatter -> owner reduction -> all-gather (gemm kEpiRsAg), then the gathered consumers."""
    torch.manual_seed(world * 1000 + T)
    N = CFG.hidden
    ranks = TensorParallel.loopback(CFG, world, "cuda", max_tokens=128)
    models = _models(ops, ranks)
    w_row = [torch.randn(N, K, device="cuda").mul_(0.05).bfloat16() for _ in ranks]
    w_col = [torch.randn(512, N, device="cuda").mul_(0.05).bfloat16() for _ in ranks]
    norm_w = torch.randn(N, device="cuda").mul_(0.1).bfloat16()
    x_ref = torch.randn(T, N, device="cuda").bfloat16()
    for tp in ranks:
        tp.x[:T].copy_(x_ref)
    x_ref = x_ref.float()
    for call in range(3):   # several calls in a row: the cumulative counters must keep agreeing
        acts = [torch.randn(T, K, device="cuda").bfloat16() for _ in ranks]
        if world == 1:
            ranks[0]._rs_ag(models[0], acts[0], w_row[0], T, phase=0)      # the production kernel, nothing to wait for
        else:
            for tp, m, a, w in zip(ranks, models, acts, w_row):
                tp._rs_ag(m, a, w, T, phase=1)
            for tp, m, a, w in zip(ranks, models, acts, w_row):
                tp._rs_ag(m, a, w, T, phase=2)
        x_ref = (x_ref + sum(a.float() @ w.float().T for a, w in zip(acts, w_row))).bfloat16().float()
        normed = _rms(x_ref)
        for tp, m, wc in zip(ranks, models, w_col):
            _close(tp.x[:T], x_ref, 1e-2)
            out = torch.empty(T, 512, device="cuda", dtype=torch.bfloat16)
            tp.gemm_gathered(m, _ws(tp), T, wc, out, EPI_STORE)
            _close(out, normed @ wc.float().T)
            act = torch.empty(T, 256, device="cuda", dtype=torch.bfloat16)
            tp.gemm_gathered(m, _ws(tp), T, wc, act, EPI_SWIGLU)
            full = normed @ wc.float().T
            _close(act, torch.nn.functional.silu(full[:, :256]) * full[:, 256:])
            nout = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            tp.gather_norm(m, _ws(tp), T, norm_w, nout)
            _close(nout, normed * (1.0 + norm_w.float()))
            m.status.check(f"rank {tp.rank} call {call}")


@pytest.mark.parametrize("world,T", [(2, 200), (4, 130)])
def test_push_partial_then_reduce_all_gather_norm(ops, world, T):
    """Prefill-sized path: gemm kEpiPushPartial, then tp_reduce_ag_norm split into its two phases."""
    torch.manual_seed(7 + world)
    N, K = CFG.hidden, 256
    ranks = TensorParallel.loopback(CFG, world, "cuda", max_tokens=256)
    models = _models(ops, ranks)
    w_row = [torch.randn(N, K, device="cuda").mul_(0.05).bfloat16() for _ in ranks]
    norm_w = torch.randn(N, device="cuda").mul_(0.1).bfloat16()
    x_ref = torch.randn(T, N, device="cuda").bfloat16()
    for tp in ranks:
        tp.x[:T].copy_(x_ref)
    x_ref = x_ref.float()
    tn = 256
    t_tiles = (T + tn - 1) // tn
    for call in range(3):
        acts = [torch.randn(T, K, device="cuda").bfloat16() for _ in ranks]
        for tp, m, a, w in zip(ranks, models, acts, w_row):
            ops.gemm_bf16_push(a, w, 1, world, tp.rank, tp.peer_bases, tp.off["recv"], tp.off["arrival_flag"],
                               m.status.tensor, False)
        normed = [torch.empty(T, N, device="cuda", dtype=torch.bfloat16) for _ in ranks]
        arrivals = world * (tp.slice // 128) * t_tiles
        for phases in (1, 2):
            for tp, m, o in zip(ranks, models, normed):
                ops.tp_reduce_ag_norm(world, tp.rank, T, tp.T_cap, N, 1, arrivals, tp.peer_bases, tp.off["recv"],
                                      tp.off["arrival_flag"], tp.off["x"], tp.off["ss"], tp.off["row_flag"], norm_w, o,
                                      EPS, True, tp.state, m.status.tensor, False, phases)
        x_ref = (x_ref + sum(a.float() @ w.float().T for a, w in zip(acts, w_row))).bfloat16().float()
        for tp, m, o in zip(ranks, models, normed):
            _close(tp.x[:T], x_ref, 1e-2)
            _close(o, _rms(x_ref) * (1.0 + norm_w.float()))
            m.status.check(f"rank {tp.rank} call {call}")


@pytest.mark.parametrize("world,T", [(2, 32), (8, 5)])
def test_push_all_then_sum_norm(ops, world, T):
    """One-shot decode path: gemm kEpiPushAll into every rank, then tp_sum_norm on every rank."""
    torch.manual_seed(11 + world)
    N, K = CFG.hidden, 512
    ranks = TensorParallel.loopback(CFG, world, "cuda", max_tokens=128, mode="oneshot")
    models = _models(ops, ranks)
    w_row = [torch.randn(N, K, device="cuda").mul_(0.05).bfloat16() for _ in ranks]
    norm_w = torch.randn(N, device="cuda").mul_(0.1).bfloat16()
    x_ref = torch.randn(T, N, device="cuda").bfloat16()
    xs = [x_ref.clone() for _ in ranks]
    x_ref = x_ref.float()
    for call in range(3):
        acts = [torch.randn(T, K, device="cuda").bfloat16() for _ in ranks]
        splits = int(ops.gemm_pick_splits(T, N, K, 5))
        for tp, m, a, w in zip(ranks, models, acts, w_row):
            ops.gemm_bf16_push_all(a, w, splits, world, tp.rank, tp.peer_bases, tp.off["recv_all"], tp.off["all_flag"],
                                   tp.one_shot_rows, tp.state, m.status.tensor, False)
        tn = 16 if T <= 16 else 32
        arrivals = world * (N // 128) * ((T + tn - 1) // tn)
        x_ref = (x_ref + sum(a.float() @ w.float().T for a, w in zip(acts, w_row))).bfloat16().float()
        for tp, m, x in zip(ranks, models, xs):
            o = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            ops.tp_sum_norm(world, tp.one_shot_rows, arrivals, tp.peer_bases[tp.rank], tp.off["recv_all"],
                            tp.off["all_flag"], x, norm_w, o, EPS, True, tp.state, m.status.tensor, False)
            _close(x, x_ref, 1e-2)
            _close(o, _rms(x_ref) * (1.0 + norm_w.float()))
            m.status.check(f"rank {tp.rank} call {call}")


def test_vocabulary_parallel_argmax_with_ties(ops):
    """Highest value wins, the lowest global id among equal values, whatever rank holds it."""
    world, T, V = 4, 6, 512
    ranks = TensorParallel.loopback(CFG, world, "cuda", max_tokens=64)
    models = _models(ops, ranks)
    torch.manual_seed(3)
    for call in range(2):
        full = torch.randn(T, world * V, device="cuda").bfloat16()
        top = full.float().max().item() + 1.0
        full[0, 3 * V + 5] = top                       # a plain winner on the last rank
        full[1, 1 * V + 9] = top; full[1, 2 * V + 1] = top      # tie across ranks: the lower rank's id wins
        full[2, 0 * V + 40] = top; full[2, 0 * V + 7] = top     # tie inside one rank
        full[3, 3 * V + 0] = top; full[3, 0 * V + 511] = top    # tie between the first and the last rank
        want = []
        for t in range(T):
            row = full[t].float()
            want.append(int((row == row.max()).nonzero()[0, 0]))
        outs = [torch.full((T,), -1, device="cuda", dtype=torch.int32) for _ in ranks]
        for phases in (1, 2):
            for tp, m, o in zip(ranks, models, outs):
                ops.tp_argmax(world, tp.rank, tp.T_cap, full[:, tp.rank * V:(tp.rank + 1) * V], tp.peer_bases,
                              tp.off["cand"], tp.off["argmax_flag"], o, tp.state, m.status.tensor, False, phases)
        for tp, m, o in zip(ranks, models, outs):
            assert o.tolist() == want, f"rank {tp.rank} call {call}: {o.tolist()} != {want}"
            m.status.check(f"rank {tp.rank}")
