"""Quantised-weight tcgen05 GEMMs (fp8 row-scale W8A8, nvfp4 block-scaled W4A4) against fp32 oracles."""
import pytest
import torch

from ninfer_fusion_b200._lib import StatusWord, load_native
from ninfer_fusion_b200.ops import quant as Q

pytestmark = pytest.mark.gpu
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2


def _act_fp8(ops, x):
    T, K = x.shape
    codes = torch.empty((T, K), dtype=torch.uint8, device="cuda")
    scale = torch.empty(T, dtype=torch.float32, device="cuda")
    ops.quant_act_fp8(x, codes, scale)
    return codes, scale


def _act_nvfp4(ops, x):
    T, K = x.shape
    codes = torch.empty((T, K // 2), dtype=torch.uint8, device="cuda")
    plane = torch.zeros(int(ops.nvfp4_act_scale_bytes(T, K)), dtype=torch.uint8, device="cuda")
    ops.quant_act_nvfp4(x, codes, plane)
    return codes, plane


@pytest.mark.parametrize("T", [1, 32, 100, 300])
def test_activation_quantisers(T):
    ops = load_native()
    torch.manual_seed(T)
    K = 1024
    x = (torch.randn(T, K, device="cuda") * torch.rand(T, 1, device="cuda") * 4).bfloat16()
    codes, scale = _act_fp8(ops, x)
    deq = Q.dequant_fp8_row(codes, scale)
    assert (deq - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    want_scale = x.float().abs().amax(-1) / 448.0
    assert torch.allclose(scale, want_scale, rtol=1e-6)
    c4, plane = _act_nvfp4(ops, x)
    deq4 = Q.dequant_nvfp4(c4, plane, 1.0, T, K)
    blk = x.float().reshape(T, K // 16, 16)
    err = (deq4.reshape(T, K // 16, 16) - blk).abs().amax(-1)
    assert (err <= 0.26 * blk.abs().amax(-1) + 1e-6).all()  # e2m1 step is at most amax/3 wide, plus the scale rounding


@pytest.mark.parametrize("qt", ["fp8", "nvfp4"])
@pytest.mark.parametrize("T,N,K,epi,splits", [
    (1, 256, 512, EPI_STORE, 1), (20, 384, 1024, EPI_RESIDUAL, 1), (32, 512, 2048, EPI_SWIGLU, 1),
    (64, 256, 2048, EPI_STORE, 4), (100, 640, 768, EPI_RESIDUAL, 1), (130, 256, 512, EPI_SWIGLU, 1),
    (300, 384, 1024, EPI_STORE, 1), (16, 5120, 5120, EPI_RESIDUAL, 3),
    # more tiles than SMs at prefill size: the persistent kernel (overlapped epilogue), ragged T
    (600, 8192, 768, EPI_STORE, 1), (777, 8192, 512, EPI_RESIDUAL, 1), (1000, 9984, 512, EPI_SWIGLU, 1)])
def test_gemm_quant_matches_oracle(qt, T, N, K, epi, splits):
    ops = load_native()
    status = StatusWord("cuda")
    torch.manual_seed(T + N)
    w = torch.randn(N, K, device="cuda") * 0.05
    x = torch.randn(T, K, device="cuda").bfloat16()
    resid = torch.randn(T, N, device="cuda").bfloat16() if epi == EPI_RESIDUAL else None
    w_rows = Q.interleave_gate_up(w) if epi == EPI_SWIGLU else w
    if qt == "fp8":
        wc, ws = Q.quantize_fp8_row(w_rows)
        xc, xs = _act_fp8(ops, x)
        w_deq, x_deq, div, code = Q.dequant_fp8_row(wc, ws), Q.dequant_fp8_row(xc, xs), 1.0, Q.QT_FP8_ROW
    else:
        wc, ws, div = Q.quantize_nvfp4(w_rows)
        xc, xs = _act_nvfp4(ops, x)
        w_deq, x_deq, code = Q.dequant_nvfp4(wc, ws, div, N, K), Q.dequant_nvfp4(xc, xs, 1.0, T, K), Q.QT_NVFP4
    out = torch.empty((T, N // 2 if epi == EPI_SWIGLU else N), dtype=torch.bfloat16, device="cuda")
    ops.gemm_quant(code, xc, xs, wc, ws, div, out, epi, resid, splits, status.tensor, False)
    torch.cuda.synchronize()
    status.check()
    acc = x_deq.double() @ w_deq.double().t()
    if epi == EPI_SWIGLU:
        t = acc.reshape(T, N // 128, 2, 64)   # tile-interleaved rows: [64 gate ; 64 up]
        want = (torch.nn.functional.silu(t[:, :, 0]) * t[:, :, 1]).reshape(T, N // 2)
    elif epi == EPI_RESIDUAL:
        want = acc + resid.double()
    else:
        want = acc
    err = (out.double() - want).abs().max().item()
    assert err <= 0.01 * want.abs().max().item() + 0.01, f"max err {err} vs scale {want.abs().max().item()}"
