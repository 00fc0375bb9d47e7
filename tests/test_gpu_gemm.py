"""tcgen05 GEMM vs an fp32 torch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_PARTIAL = 0, 1, 2, 3


def _mk(T, N, K, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    return x, w


def _check(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("T", [1, 7, 16, 32, 48, 64, 100, 128, 300, 513])
@pytest.mark.parametrize("N,K", [(256, 512), (384, 192), (5120, 1024)])
def test_gemm_store(ops, status, T, N, K):
    x, w = _mk(T, N, K)
    out = torch.full((T, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, out, EPI_STORE, None, None, None, 1, status.tensor, False)
    _check(out, x.float() @ w.float().t())


def test_gemm_store_ragged_n_and_k(ops, status):
    # N not a multiple of 128, K not a multiple of 64: TMA zero-fills the tails
    x, w = _mk(20, 16480 // 8, 200)
    out = torch.empty((20, w.shape[0]), device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, out, EPI_STORE, None, None, None, 1, status.tensor, False)
    _check(out, x.float() @ w.float().t())


def test_gemm_strided_views_and_bias(ops, status):
    x_full, w = _mk(33, 256, 1024)
    x = x_full[:, :512]
    w = w[:, :512]
    out_full = torch.zeros((33, 512), device="cuda", dtype=torch.bfloat16)
    out = out_full[:, 128:384]
    bias = torch.randn(256, device="cuda")
    ops.gemm_bf16(x, w, out, EPI_STORE, None, bias, None, 1, status.tensor, False)
    _check(out, x.float() @ w.float().t() + bias)
    assert out_full[:, :128].abs().max().item() == 0 and out_full[:, 384:].abs().max().item() == 0


@pytest.mark.parametrize("T", [1, 32, 130])
def test_gemm_residual(ops, status, T):
    x, w = _mk(T, 512, 768)
    resid = torch.randn(T, 512, device="cuda").to(torch.bfloat16)
    out = resid.clone()
    ops.gemm_bf16(x, w, out, EPI_RESIDUAL, out, None, None, 1, status.tensor, False)
    _check(out, resid.float() + x.float() @ w.float().t())


@pytest.mark.parametrize("T", [1, 32, 64, 257])
@pytest.mark.parametrize("inter", [64, 192, 1024])
def test_gemm_swiglu(ops, status, T, inter):
    x, w = _mk(T, 2 * inter, 512)
    out = torch.empty((T, inter), device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, out, EPI_SWIGLU, None, None, None, 1, status.tensor, False)
    gu = x.float() @ w.float().t()
    _check(out, torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:])


@pytest.mark.parametrize("T,splits", [(1, 4), (32, 7), (64, 3)])
def test_gemm_splitk_and_reduce(ops, status, T, splits):
    N, K = 640, 64 * 40
    x, w = _mk(T, N, K)
    part = torch.full((splits * T * N,), float("nan"), device="cuda")
    ops.gemm_bf16(x, w, None, EPI_PARTIAL, None, None, part, splits, status.tensor, False)
    ref = x.float() @ w.float().t()
    _check(part.view(splits, T, N).sum(0), ref, 1e-3)
    # fused reduce + residual + rmsnorm
    resid = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    nw = (torch.randn(N, device="cuda") * 0.1).to(torch.bfloat16)
    r_out = torch.empty_like(resid)
    normed = torch.empty_like(resid)
    ops.add_rmsnorm(part, splits, None, resid, r_out, nw, normed, T, N, 1e-6, True, False)
    xr = (resid.float() + ref).to(torch.bfloat16).float()
    _check(r_out, xr, 1e-2)
    nr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())
    _check(normed, nr, 2e-2)


def test_pick_splits_covers_k(ops):
    for T, N, K in [(32, 5120, 17408), (32, 5120, 6144), (1, 5120, 6144), (64, 248320, 5120), (300, 5120, 6144)]:
        s = int(ops.gemm_pick_splits(T, N, K, EPI_PARTIAL))
        nkb = (K + 63) // 64
        per = (nkb + s - 1) // s
        assert 1 <= s <= 8 and (nkb + per - 1) // per == s
    for T, N, K, epi in [(32, 5120, 17408, EPI_RESIDUAL), (32, 2060, 5120, EPI_STORE), (1, 34816, 5120, EPI_SWIGLU)]:
        s = int(ops.gemm_pick_splits(T, N, K, epi))
        assert 1 <= s <= 8


def test_gemm_pdl_chain(ops, status):
    """Back-to-back launches with programmatic dependent launch read each other's output."""
    x, w1 = _mk(32, 512, 512)
    _, w2 = _mk(32, 256, 512, seed=1)
    h = torch.empty((32, 512), device="cuda", dtype=torch.bfloat16)
    out = torch.empty((32, 256), device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        ops.gemm_bf16(x, w1, h, EPI_STORE, None, None, None, 1, status.tensor, True)
        ops.gemm_bf16(h, w2, out, EPI_STORE, None, None, None, 1, status.tensor, True)
    ref_h = (x.float() @ w1.float().t()).to(torch.bfloat16).float()
    _check(out, ref_h @ w2.float().t())


@pytest.mark.parametrize("T,splits", [(1, 8), (16, 5), (32, 2), (32, 6), (32, 3), (64, 2), (100, 2)])
@pytest.mark.parametrize("epi", [EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU])
def test_gemm_cluster_splitk(ops, status, T, splits, epi):
    """Split-K inside a thread-block cluster: peers hand fp32 tiles to the leader through DSMEM."""
    N, K = 512, 64 * 36 + 8
    x, w = _mk(T, N, K, seed=3)
    ref = x.float() @ w.float().t()
    if epi == EPI_SWIGLU:
        out = torch.full((T, N // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(x, w, out, epi, None, None, None, splits, status.tensor, False)
        _check(out, torch.nn.functional.silu(ref[:, : N // 2]) * ref[:, N // 2:])
    elif epi == EPI_RESIDUAL:
        resid = torch.randn(T, N, device="cuda").to(torch.bfloat16)
        out = resid.clone()
        ops.gemm_bf16(x, w, out, epi, out, None, None, splits, status.tensor, False)
        _check(out, resid.float() + ref)
    else:
        out = torch.full((T, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(x, w, out, epi, None, None, None, splits, status.tensor, True)
        _check(out, ref)


def test_gemm_cluster_splitk_is_deterministic(ops, status):
    x, w = _mk(32, 5120, 6144, seed=4)
    outs = []
    for _ in range(3):
        out = torch.empty((32, 5120), device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(x, w, out, EPI_STORE, None, None, None, 4, status.tensor, False)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    _check(outs[0], x.float() @ w.float().t())


@pytest.mark.parametrize("T", [300, 777, 2048])
def test_gemm_persistent_prefill_kernel(ops, status, T):
    """More output tiles than SMs at TN = 256: the persistent kernel (epilogue overlapped with the next main loop)
    with every plain epilogue, ragged T / N / K, bias + GELU, in-place residual; checked tile by tile."""
    # store + bias + GELU(tanh), N and K not multiples of the tile
    x, w = _mk(T, 20040, 1096, seed=1)
    bias = torch.randn(20040, device="cuda")
    out = torch.full((T, 20040), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, out, EPI_STORE, None, bias, None, 1, status.tensor, False, 1)
    ref = torch.nn.functional.gelu(x.float() @ w.float().t() + bias, approximate="tanh")
    _check(out, ref)
    assert not torch.isnan(out).any()
    # in-place residual
    x, w = _mk(T, 19200, 512, seed=2)
    resid = torch.randn(T, 19200, device="cuda").to(torch.bfloat16)
    out = resid.clone()
    ops.gemm_bf16(x, w, out, EPI_RESIDUAL, out, None, None, 1, status.tensor, False)
    _check(out, resid.float() + x.float() @ w.float().t())
    # SwiGLU with [gate; up] parent
    inter = 9792
    x, w = _mk(T, 2 * inter, 640, seed=3)
    out = torch.full((T, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, out, EPI_SWIGLU, None, None, None, 1, status.tensor, False)
    gu = x.float() @ w.float().t()
    _check(out, torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:])
    assert not torch.isnan(out).any()
    # twice in a row on the same stream (barrier phases restart per launch), PDL attribute set
    out2 = torch.empty_like(out)
    ops.gemm_bf16(x, w, out2, EPI_SWIGLU, None, None, None, 1, status.tensor, True)
    assert torch.equal(out, out2)
    status.check("persistent gemm")


@pytest.mark.parametrize("T,N,K,C", [(32, 1024, 512, 512), (5, 640, 256, 384), (64, 2048, 1024, 1280)])
def test_gemm_conv_epilogue_matches_separate_conv(ops, status, T, N, K, C):
    """Decode conv + SiLU + history roll inside the store epilogue = GEMM followed by the stand-alone conv kernel."""
    torch.manual_seed(T + N)
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").mul_(0.05).bfloat16()
    conv_w = torch.randn(C, 4, device="cuda").mul_(0.3).bfloat16()
    n_slots = T + 3
    slots = torch.randperm(n_slots, device="cuda")[:T].int()
    state0 = torch.randn(n_slots, 3, C, device="cuda").bfloat16()
    splits = int(ops.gemm_pick_splits(T, N, K, 0))
    # separate kernels
    proj = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, proj, 0, None, None, None, splits, status.tensor, False)
    st_a, out_a = state0.clone(), torch.empty(T, C, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(T + 1, device="cuda", dtype=torch.int32)
    seq = torch.arange(T, device="cuda", dtype=torch.int32)
    ops.causal_conv1d_silu(proj, 0, C, conv_w, cu, seq, slots, st_a, out_a, True, True, False)
    # fused
    proj_b = torch.zeros(T, N, device="cuda", dtype=torch.bfloat16)
    st_b, out_b = state0.clone(), torch.empty(T, C, device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, proj_b, 0, None, None, None, splits, status.tensor, False, 0, conv_w, st_b, slots, out_b)
    torch.cuda.synchronize()
    assert torch.equal(st_a, st_b)                                  # the history is a copy of bf16 values
    assert torch.equal(proj[:, C:], proj_b[:, C:])                  # columns past the conv channels: plain output
    torch.testing.assert_close(out_b.float(), out_a.float(), rtol=1e-2, atol=1e-2)
    # and against the definition
    hist = state0[slots.long()].float()                             # [T, 3, C]
    taps = torch.cat([hist, proj[:, None, :C].float()], dim=1)      # [T, 4, C]
    ref = torch.nn.functional.silu((taps * conv_w.float().T[None]).sum(1))
    torch.testing.assert_close(out_b.float(), ref, rtol=2e-2, atol=2e-2)
