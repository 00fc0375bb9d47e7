"""Weight quantisers and de-quantisers (torch, any device) for the quantised-weight GEMMs.

Numeric contracts (docs/maintainer/tensor-formats.md:279-353): NVFP4 ``W = e2m1 * e4m3 / d_w`` with one
e4m3 scale per 16 values stored in 128x4 tiles; FP8 ``w = e4m3 * row_scale``.  The planes produced here
are the operands of ``torch.ops.nfb200.gemm_quant`` and the payloads of the artifact layouts
``blockscale-k16-m128x4-v1`` / ``row-scale-v1`` (artifact/layouts.py holds the byte-level container code).
"""
from __future__ import annotations

from typing import Tuple

import torch

QT_FP8_ROW, QT_NVFP4 = 1, 2
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto the e2m1 grid; returns uint8 codes (bit 3 = sign)."""
    a = x.abs()
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
    up_on_tie = torch.tensor([False, True, False, True, False, True, False], device=x.device)
    idx = torch.zeros_like(a, dtype=torch.uint8)
    for b, up in zip(bounds, up_on_tie):
        idx += ((a >= b) if bool(up) else (a > b)).to(torch.uint8)
    return idx | (torch.signbit(x).to(torch.uint8) << 3)


def e2m1_values(codes: torch.Tensor) -> torch.Tensor:
    mag = _E2M1.to(codes.device)[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


def sf_tile_offsets(rows: int, K: int, device) -> torch.Tensor:
    """Byte offset of scale (row, 16-value block) in the 128x4-tiled plane, as an int64 [rows, K/16] tensor."""
    r = torch.arange(rows, device=device)[:, None]
    g = torch.arange(K // 16, device=device)[None, :]
    return ((r // 128) * (K // 64) + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4


def quantize_nvfp4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, float]:
    """w [N, K] -> (packed codes uint8 [N, K/2], scale plane uint8 [ceil(N/128) * K/64 * 512], d_w)."""
    N, K = w.shape
    g = w.float().reshape(N, K // 16, 16)
    amax = g.abs().amax(-1)
    gmax = float(amax.max())
    d_w = 448.0 * 6.0 / gmax if gmax > 0 else 1.0
    sf = (amax * d_w / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    s = sf.float()
    inv = torch.where(s > 0, d_w / torch.where(s > 0, s, torch.ones_like(s)), torch.zeros_like(s))
    codes = e2m1_codes(g * inv[..., None]).reshape(N, K)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    plane = torch.zeros(((N + 127) // 128) * (K // 64) * 512, dtype=torch.uint8, device=w.device)
    plane[sf_tile_offsets(N, K, w.device).reshape(-1)] = sf.view(torch.uint8).reshape(-1)
    return packed.contiguous(), plane, d_w


def quantize_nvfp4_prepare(w: torch.Tensor, rows_per_step: int = 16384) -> Tuple[torch.Tensor, torch.Tensor, float]:
    """quantize_nvfp4 for large matrices: the global divisor comes from one pass over the matrix, then the
    rows are encoded in slabs (multiples of 128 rows) to bound the temporary memory."""
    N, K = w.shape
    gmax = float(w.abs().amax())
    d_w = 448.0 * 6.0 / gmax if gmax > 0 else 1.0
    packed = torch.empty((N, K // 2), dtype=torch.uint8, device=w.device)
    plane = torch.zeros(((N + 127) // 128) * (K // 64) * 512, dtype=torch.uint8, device=w.device)
    tile_bytes = (K // 64) * 512
    for r0 in range(0, N, rows_per_step):
        r1 = min(N, r0 + rows_per_step)
        g = w[r0:r1].float().reshape(r1 - r0, K // 16, 16)
        amax = g.abs().amax(-1)
        sf = (amax * d_w / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
        s = sf.float()
        inv = torch.where(s > 0, d_w / torch.where(s > 0, s, torch.ones_like(s)), torch.zeros_like(s))
        codes = e2m1_codes(g * inv[..., None]).reshape(r1 - r0, K)
        packed[r0:r1] = codes[:, 0::2] | (codes[:, 1::2] << 4)
        off = sf_tile_offsets(r1 - r0, K, w.device).reshape(-1) + (r0 // 128) * tile_bytes
        plane[off] = sf.view(torch.uint8).reshape(-1)
    return packed, plane, d_w


def dequant_nvfp4(packed: torch.Tensor, plane: torch.Tensor, divisor: float, rows: int, K: int) -> torch.Tensor:
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(rows, K)
    sf = plane[sf_tile_offsets(rows, K, packed.device).reshape(-1)].view(torch.float8_e4m3fn).float().reshape(rows, K // 16)
    return (e2m1_values(codes).reshape(rows, K // 16, 16) * sf[..., None]).reshape(rows, K) / divisor


def quantize_fp8_row(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [N, K] -> (e4m3 codes uint8 [N, K], fp32 row scales [N])."""
    amax = w.float().abs().amax(-1)
    scale = (amax / 448.0).clamp(min=1e-12)
    codes = (w.float() / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    return codes.contiguous(), scale.float()


def dequant_fp8_row(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return codes.view(torch.float8_e4m3fn).float() * scale[:, None]


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """[gate; up] rows -> 128-row tiles of [64 gate rows ; 64 up rows] (what the quantised SwiGLU epilogue reads)."""
    two_i, K = w.shape
    i = two_i // 2
    if i % 64:
        raise ValueError("intermediate size must be a multiple of 64")
    gate, up = w[:i].reshape(i // 64, 64, K), w[i:].reshape(i // 64, 64, K)
    return torch.cat([gate, up], dim=1).reshape(two_i, K).contiguous()


def deinterleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """Inverse of interleave_gate_up."""
    two_i, K = w.shape
    t = w.reshape(two_i // 128, 2, 64, K)
    return torch.cat([t[:, 0].reshape(two_i // 2, K), t[:, 1].reshape(two_i // 2, K)], dim=0).contiguous()


def fake_quant_nvfp4(x: torch.Tensor) -> torch.Tensor:
    """Activation quantisation of the W4A4 path as a value map: per 16 values scale = e4m3(amax / 6), e2m1 codes."""
    T, K = x.shape
    g = bf16(x).reshape(T, K // 16, 16)
    sf = (g.abs().amax(-1) / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn).float()
    safe = torch.where(sf > 0, sf, torch.ones_like(sf))
    q = e2m1_values(e2m1_codes(torch.where(sf[..., None] > 0, g / safe[..., None], torch.zeros_like(g))))
    return (q * sf[..., None]).reshape(T, K)


def fake_quant_fp8(x: torch.Tensor) -> torch.Tensor:
    """Activation quantisation of the W8A8 path as a value map: per token scale = amax / 448, e4m3 codes."""
    xb = bf16(x)
    scale = (xb.abs().amax(-1, keepdim=True) / 448.0).clamp(min=1e-12)
    return (xb / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * scale


def bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def quantize_fp8_block128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [..., N, K] (N, K multiples of 128) -> (e4m3 codes uint8 [..., N, K], fp32 scales [..., N/128, K/128])."""
    *lead, N, K = w.shape
    blocks = w.float().reshape(*lead, N // 128, 128, K // 128, 128)
    scale = (blocks.abs().amax(dim=(-3, -1)) / 448.0).clamp(min=1e-12)
    codes = (blocks / scale[..., :, None, :, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    return codes.reshape(*lead, N, K).contiguous(), scale.float().contiguous()


def dequant_fp8_block128(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    *lead, N, K = codes.shape
    v = codes.view(torch.float8_e4m3fn).float().reshape(*lead, N // 128, 128, K // 128, 128)
    return (v * scale[..., :, None, :, None]).reshape(*lead, N, K)


def fake_quant_fp8_block128_rows(x: torch.Tensor) -> torch.Tensor:
    """Activation quantisation of the fp8 block-scaled expert path as a value map: per row and 128-wide k-block."""
    T, K = x.shape
    g = bf16(x).reshape(T, K // 128, 128)
    scale = (g.abs().amax(-1, keepdim=True) / 448.0).clamp(min=1e-12)
    return ((g / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * scale).reshape(T, K)
