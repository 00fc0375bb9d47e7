"""Registered tensor formats and storage layouts of the `.ninfer` v2 container.

Byte rules follow the reference's layout registry (docs/maintainer/storage-layouts.md:82-325,
docs/maintainer/tensor-formats.md:279-353): `contiguous-le-v1` for direct words,
`row-split-k128-v1` for the grouped signed-integer formats (base / high-bit / fp16-scale planes,
256-byte plane alignment), `blockscale-k16-m128x4-v1` for NVFP4 (row-major packed E2M1 codes, a
128x4-tile swizzled E4M3 scale plane, trailing fp32 divisor) and `row-scale-v1` for fp8 rows with a
bf16 multiplier.  One layout is new here and has its own identity:
`blockscale-128x128-f32-v1` for `FP8_E4M3FN_BLOCK128_F32S` (fp8 codes with one fp32 scale per
128x128 block), the storage of the expert banks in the MoE configuration.

Every encoder returns the exact payload bytes; every decoder recovers the logical words (codes and
scales) and, on request, the represented fp32 weights.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Sequence, Tuple

import numpy as np
import torch

OBJECT_ALIGNMENT = 256

DIRECT_FORMATS = {"BF16": 2, "FP32": 4, "I32": 4}
GROUP_FORMATS = {  # name -> (code bits, group, base bytes / group, high bytes / group, qmax)
    "Q4G64_F16S": (4, 64, 32, 0, 7),
    "Q5G64_F16S": (5, 64, 32, 8, 15),
    "Q6G64_F16S": (6, 64, 32, 16, 31),
    "W8G32_F16S": (8, 32, 32, 0, 127),
}
LAYOUTS: Dict[str, frozenset] = {
    "contiguous-le-v1": frozenset(DIRECT_FORMATS),
    "row-split-k128-v1": frozenset(GROUP_FORMATS),
    "blockscale-k16-m128x4-v1": frozenset({"NVFP4"}),
    "row-scale-v1": frozenset({"FP8_E4M3FN_ROW_BF16S"}),
    "blockscale-128x128-f32-v1": frozenset({"FP8_E4M3FN_BLOCK128_F32S"}),
}
FORMATS = frozenset().union(*LAYOUTS.values())
ENCODINGS = frozenset({"raw-bytes-v1"})


def align_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def default_layout(fmt: str) -> str:
    for name, fmts in LAYOUTS.items():
        if fmt in fmts:
            return name
    raise ValueError(f"unknown tensor format {fmt}")


def encoded_size(fmt: str, layout: str, shape: Sequence[int]) -> int:
    if layout not in LAYOUTS or fmt not in LAYOUTS[layout]:
        raise ValueError(f"format {fmt} is not stored in layout {layout}")
    n_el = int(np.prod(shape)) if len(shape) else 1
    if layout == "contiguous-le-v1":
        return n_el * DIRECT_FORMATS[fmt]
    if len(shape) != 2:
        raise ValueError(f"{layout} stores rank-2 matrices only")
    N, K = shape
    if layout == "row-split-k128-v1":
        _, G, B, H, _ = GROUP_FORMATS[fmt]
        gpr = align_up(K, 128) // G
        base, high, scale = N * gpr * B, N * gpr * H, N * gpr * 2
        return align_up(base, 256) + align_up(high, 256) + scale
    if layout == "blockscale-k16-m128x4-v1":
        if N % 128 or K % 64:
            raise ValueError("NVFP4 needs N % 128 == 0 and K % 64 == 0")
        return align_up(N * K // 2, 256) + N * K // 16 + 4
    if layout == "row-scale-v1":
        return align_up(N * K, 256) + N * 2
    if layout == "blockscale-128x128-f32-v1":
        return align_up(N * K, 256) + ((N + 127) // 128) * ((K + 127) // 128) * 4
    raise ValueError(layout)


# ---------------------------------------------------------------------------- numeric helpers
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.array(b, dtype=np.uint8, copy=True)).view(torch.float8_e4m3fn).float().numpy()


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).clamp(-448.0, 448.0)
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def f32_to_e2m1_codes(x: np.ndarray) -> np.ndarray:
    a = np.abs(x)
    bounds = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    up_on_tie = np.array([0, 1, 0, 1, 0, 1, 0], dtype=bool)
    idx = np.zeros(a.shape, dtype=np.uint8)
    for b, up in zip(bounds, up_on_tie):
        idx += (a >= b) if up else (a > b)
    return idx | (np.signbit(x).astype(np.uint8) << 3)


def nvfp4_scale_offset(n: np.ndarray, g: np.ndarray, K: int) -> np.ndarray:
    """Byte offset of scale word (row n, K-group g) inside the swizzled scale plane."""
    k_tiles = K // 64
    row_tile, row_inner = n // 128, n % 128
    return (row_tile * k_tiles + g // 4) * 512 + (row_inner % 32) * 16 + (row_inner // 32) * 4 + g % 4


# ---------------------------------------------------------------------------- quantisers (fp32 -> logical words)
def quantize_group_int(w: np.ndarray, fmt: str) -> Tuple[np.ndarray, np.ndarray]:
    """Symmetric per-group quantisation: scale = fp16(amax / qmax), code = clamp(rne(w / scale))."""
    bits, G, _, _, qmax = GROUP_FORMATS[fmt]
    N, K = w.shape
    Kp = align_up(K, 128)
    wp = np.zeros((N, Kp), dtype=np.float32)
    wp[:, :K] = w
    g = wp.reshape(N, Kp // G, G)
    scale = (np.abs(g).max(-1) / qmax).astype(np.float16)
    s32 = scale.astype(np.float32)
    inv = np.where(s32 > 0, 1.0 / np.where(s32 > 0, s32, 1), 0).astype(np.float32)
    lo = -qmax if fmt == "W8G32_F16S" else -(qmax + 1)
    codes = np.clip(np.rint(g * inv[..., None]), lo, qmax).astype(np.int8)
    logical_groups = (K + G - 1) // G
    scale[:, logical_groups:] = 0
    return codes.reshape(N, Kp), scale


def quantize_nvfp4(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray, np.float32]:
    """codes [N,K] (4-bit words), scales [N,K/16] e4m3 words, divisor d_w so that W = e2m1 * e4m3 / d_w."""
    N, K = w.shape
    g = w.reshape(N, K // 16, 16).astype(np.float32)
    amax = np.abs(g).max(-1)
    gmax = float(amax.max()) if amax.size else 0.0
    d_w = np.float32(448.0 * 6.0 / gmax) if gmax > 0 else np.float32(1.0)
    scale_words = f32_to_e4m3(amax * d_w / 6.0)
    s = e4m3_to_f32(scale_words)
    inv = np.where(s > 0, d_w / np.where(s > 0, s, 1), 0).astype(np.float32)
    codes = f32_to_e2m1_codes(g * inv[..., None]).reshape(N, K)
    return codes, scale_words, d_w


def quantize_fp8_row(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    amax = np.abs(w).max(-1)
    scale = torch.from_numpy((amax / 448.0).astype(np.float32)).to(torch.bfloat16)
    s32 = scale.float().numpy()
    inv = np.where(s32 > 0, 1.0 / np.where(s32 > 0, s32, 1), 0).astype(np.float32)
    return f32_to_e4m3(w * inv[:, None]), scale.view(torch.int16).numpy().view(np.uint16)


def quantize_fp8_block128(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = np.zeros((nb * 128, kb * 128), dtype=np.float32)
    wp[:N, :K] = w
    blocks = wp.reshape(nb, 128, kb, 128)
    scale = (np.abs(blocks).max(axis=(1, 3)) / 448.0).astype(np.float32)
    inv = np.where(scale > 0, 1.0 / np.where(scale > 0, scale, 1), 0).astype(np.float32)
    codes = f32_to_e4m3((blocks * inv[:, None, :, None]).reshape(nb * 128, kb * 128)[:N, :K])
    return codes, scale


# ---------------------------------------------------------------------------- encoders (logical words -> payload bytes)
def encode_direct(t: torch.Tensor, fmt: str) -> bytes:
    dt = {"BF16": torch.bfloat16, "FP32": torch.float32, "I32": torch.int32}[fmt]
    t = t.detach().to("cpu", dt).contiguous()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def encode_row_split(codes: np.ndarray, scale: np.ndarray, fmt: str, K: int) -> bytes:
    bits, G, B, H, _ = GROUP_FORMATS[fmt]
    N, Kp = codes.shape
    u = codes.astype(np.int16) & ((1 << bits) - 1)
    if fmt == "W8G32_F16S":
        base = u.astype(np.uint8).tobytes()
    else:
        lo = (u & 0xF).astype(np.uint8)
        base = (lo[:, 0::2] | (lo[:, 1::2] << 4)).astype(np.uint8).tobytes()
    high = b""
    if H:
        hb = bits - 4
        hv = ((u >> 4) & ((1 << hb) - 1)).astype(np.uint8)          # [N, Kp]
        bitsarr = np.stack([(hv >> j) & 1 for j in range(hb)], axis=-1).reshape(N, -1)  # lane-major, bit 4 first
        high = np.packbits(bitsarr, axis=-1, bitorder="little").tobytes()
    out = bytearray(base)
    out += bytes(align_up(len(out), 256) - len(out))
    out += high
    out += bytes(align_up(len(out), 256) - len(out))
    out += scale.astype(np.float16).tobytes()
    return bytes(out)


def decode_row_split(payload: bytes, fmt: str, shape: Sequence[int]) -> Tuple[np.ndarray, np.ndarray]:
    bits, G, B, H, _ = GROUP_FORMATS[fmt]
    N, K = shape
    Kp = align_up(K, 128)
    gpr = Kp // G
    base_bytes, high_bytes = N * gpr * B, N * gpr * H
    high_off = align_up(base_bytes, 256)
    scale_off = high_off + align_up(high_bytes, 256)
    buf = np.frombuffer(payload, dtype=np.uint8)
    base = buf[:base_bytes]
    if fmt == "W8G32_F16S":
        codes = base.view(np.int8).reshape(N, Kp).astype(np.int16)
    else:
        u = np.empty((N, Kp), dtype=np.int16)
        b2 = base.reshape(N, Kp // 2)
        u[:, 0::2] = b2 & 0xF
        u[:, 1::2] = b2 >> 4
        if H:
            hb = bits - 4
            hbits = np.unpackbits(buf[high_off:high_off + high_bytes].reshape(N, -1), axis=-1, bitorder="little")
            hbits = hbits.reshape(N, Kp, hb).astype(np.int16)
            for j in range(hb):
                u |= hbits[:, :, j] << (4 + j)
        codes = np.where(u >= (1 << (bits - 1)), u - (1 << bits), u).astype(np.int16)
    scale = buf[scale_off:scale_off + N * gpr * 2].view(np.float16).reshape(N, gpr)
    return codes, scale


def dequant_row_split(codes: np.ndarray, scale: np.ndarray, fmt: str, K: int) -> np.ndarray:
    G = GROUP_FORMATS[fmt][1]
    N, Kp = codes.shape
    w = codes.reshape(N, Kp // G, G).astype(np.float32) * scale.astype(np.float32)[..., None]
    return w.reshape(N, Kp)[:, :K]


def encode_nvfp4(codes: np.ndarray, scale_words: np.ndarray, d_w: np.float32) -> bytes:
    N, K = codes.shape
    packed = (codes[:, 0::2] & 0xF) | ((codes[:, 1::2] & 0xF) << 4)
    out = bytearray(packed.astype(np.uint8).tobytes())
    out += bytes(align_up(len(out), 256) - len(out))
    plane = np.zeros(N * K // 16, dtype=np.uint8)
    n, g = np.meshgrid(np.arange(N), np.arange(K // 16), indexing="ij")
    plane[nvfp4_scale_offset(n, g, K)] = scale_words
    out += plane.tobytes()
    out += np.float32(d_w).tobytes()
    return bytes(out)


def decode_nvfp4(payload: bytes, shape: Sequence[int]) -> Tuple[np.ndarray, np.ndarray, np.float32]:
    N, K = shape
    buf = np.frombuffer(payload, dtype=np.uint8)
    packed = buf[: N * K // 2].reshape(N, K // 2)
    codes = np.empty((N, K), dtype=np.uint8)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    soff = align_up(N * K // 2, 256)
    plane = buf[soff: soff + N * K // 16]
    n, g = np.meshgrid(np.arange(N), np.arange(K // 16), indexing="ij")
    scale_words = plane[nvfp4_scale_offset(n, g, K)]
    d_w = buf[soff + N * K // 16: soff + N * K // 16 + 4].view(np.float32)[0]
    return codes, scale_words, d_w


def dequant_nvfp4(codes: np.ndarray, scale_words: np.ndarray, d_w: np.float32) -> np.ndarray:
    N, K = codes.shape
    v = E2M1_VALUES[codes & 7] * np.where(codes & 8, -1.0, 1.0).astype(np.float32)
    s = e4m3_to_f32(scale_words)
    return (v.reshape(N, K // 16, 16) * s[..., None] / np.float32(d_w)).reshape(N, K)


def encode_fp8_row(code_words: np.ndarray, scale_bf16_words: np.ndarray) -> bytes:
    out = bytearray(code_words.astype(np.uint8).tobytes())
    out += bytes(align_up(len(out), 256) - len(out))
    out += scale_bf16_words.astype(np.uint16).tobytes()
    return bytes(out)


def decode_fp8_row(payload: bytes, shape: Sequence[int]) -> Tuple[np.ndarray, np.ndarray]:
    N, K = shape
    buf = np.frombuffer(payload, dtype=np.uint8)
    soff = align_up(N * K, 256)
    return buf[: N * K].reshape(N, K), buf[soff: soff + 2 * N].view(np.uint16)


def dequant_fp8_row(code_words: np.ndarray, scale_bf16_words: np.ndarray) -> np.ndarray:
    s = torch.from_numpy(scale_bf16_words.astype(np.int16)).view(torch.bfloat16).float().numpy()
    return e4m3_to_f32(code_words) * s[:, None]


def encode_fp8_block128(code_words: np.ndarray, scales: np.ndarray) -> bytes:
    out = bytearray(code_words.astype(np.uint8).tobytes())
    out += bytes(align_up(len(out), 256) - len(out))
    out += scales.astype(np.float32).tobytes()
    return bytes(out)


def decode_fp8_block128(payload: bytes, shape: Sequence[int]) -> Tuple[np.ndarray, np.ndarray]:
    N, K = shape
    buf = np.frombuffer(payload, dtype=np.uint8)
    soff = align_up(N * K, 256)
    nb, kb = (N + 127) // 128, (K + 127) // 128
    return buf[: N * K].reshape(N, K), buf[soff: soff + nb * kb * 4].view(np.float32).reshape(nb, kb)


def dequant_fp8_block128(code_words: np.ndarray, scales: np.ndarray) -> np.ndarray:
    N, K = code_words.shape
    s = np.repeat(np.repeat(scales, 128, axis=0)[:N], 128, axis=1)[:, :K]
    return e4m3_to_f32(code_words) * s


def encode_tensor(t: torch.Tensor, fmt: str) -> Tuple[bytes, str]:
    """Quantise (where the format quantises) and encode an fp tensor; returns (payload, layout)."""
    layout = default_layout(fmt)
    if layout == "contiguous-le-v1":
        return encode_direct(t, fmt), layout
    w = t.detach().float().cpu().numpy()
    if layout == "row-split-k128-v1":
        codes, scale = quantize_group_int(w, fmt)
        return encode_row_split(codes, scale, fmt, w.shape[1]), layout
    if layout == "blockscale-k16-m128x4-v1":
        return encode_nvfp4(*quantize_nvfp4(w)), layout
    if layout == "row-scale-v1":
        return encode_fp8_row(*quantize_fp8_row(w)), layout
    return encode_fp8_block128(*quantize_fp8_block128(w)), layout


def decode_tensor(payload: bytes, fmt: str, layout: str, shape: Sequence[int]) -> torch.Tensor:
    """Represented values of a stored tensor (fp32 for quantised formats, native dtype for direct ones)."""
    if len(payload) != encoded_size(fmt, layout, shape):
        raise ValueError("payload length does not match the layout's encoded size")
    if layout == "contiguous-le-v1":
        dt = {"BF16": torch.bfloat16, "FP32": torch.float32, "I32": torch.int32}[fmt]
        return torch.frombuffer(bytearray(payload), dtype=dt).reshape(tuple(shape)).clone()
    if layout == "row-split-k128-v1":
        codes, scale = decode_row_split(payload, fmt, shape)
        return torch.from_numpy(dequant_row_split(codes, scale, fmt, shape[1]).copy())
    if layout == "blockscale-k16-m128x4-v1":
        return torch.from_numpy(dequant_nvfp4(*decode_nvfp4(payload, shape)).astype(np.float32))
    if layout == "row-scale-v1":
        return torch.from_numpy(dequant_fp8_row(*decode_fp8_row(payload, shape)).astype(np.float32))
    return torch.from_numpy(dequant_fp8_block128(*decode_fp8_block128(payload, shape)).astype(np.float32))
