"""Cold-slot codecs: the lossy requantised slot for retired KV pages and the lossless entropy stage on top of it.

* ``pack_cold_slot`` / ``restore_cold_slot``: one (page, head, plane) of KV values -> 16-byte header + packed E2M1
  nibbles + E4M3 scales per 16 values (9232 bytes for a 64-token page of head_dim 256), and back; int8 group-64 planes
  go through ``requant_int8_g64`` / ``restore_int8_g64``.  Reference: include/ninfer/ops/cold_i8.h (slot layout and
  the lossy-by-construction contract), src/ops/kv_cache entropy_cold_requant.
* ``rans_encode`` / ``rans_decode``: static-table range-ANS over 4-bit or 8-bit symbols with a byte budget (native
  coder in csrc/runtime/rans_codec.cpp, byte-identical Python twin here).  Reference:
  include/ninfer/ops/entropy_nvfp4_slot.h (rANS slot coder with budgeted streams).
* ``save_cold`` / ``load_cold``: the disk tier's file format, each tensor coded when that saves space.
"""
from __future__ import annotations

import ctypes
import io
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..artifact import layouts as L

PROB_BITS = 12
PROB_SCALE = 1 << PROB_BITS
LOW = 1 << 23
SLOT_MAGIC = 0x31534C43   # "CLS1"
SLOT_HEADER = 16


# ---------------------------------------------------------------------------------------------- native coder
def _load_lib():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")
    if not os.path.exists(path) or os.environ.get("NFB200_PY_RANS") == "1":
        return None
    try:
        import torch  # noqa: F401  (the library links against torch's shared objects)
        lib = ctypes.CDLL(path)
        u8p = ctypes.POINTER(ctypes.c_uint8)
        lib.nfb200_rans_bound.restype = ctypes.c_int64
        lib.nfb200_rans_bound.argtypes = [ctypes.c_int64, ctypes.c_int]
        lib.nfb200_rans_encode.restype = ctypes.c_int64
        lib.nfb200_rans_encode.argtypes = [u8p, ctypes.c_int64, ctypes.c_int, u8p, ctypes.c_int64]
        lib.nfb200_rans_decode.restype = ctypes.c_int64
        lib.nfb200_rans_decode.argtypes = [u8p, ctypes.c_int64, u8p, ctypes.c_int64]
        return lib
    except (OSError, AttributeError):
        return None


_LIB = _load_lib()


def native_available() -> bool:
    return _LIB is not None


def rans_bound(n_bytes: int, bits: int) -> int:
    return 10 + 2 * (1 << bits) + n_bytes + n_bytes // 64 + 16


def _as_u8(data) -> np.ndarray:
    if isinstance(data, torch.Tensor):
        return data.detach().cpu().contiguous().view(torch.uint8).reshape(-1).numpy()
    if isinstance(data, np.ndarray):
        return np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    return np.frombuffer(bytes(data), dtype=np.uint8)


# ---------------------------------------------------------------------------------------------- Python twin
def _symbols(src: np.ndarray, bits: int) -> np.ndarray:
    if bits == 8:
        return src
    out = np.empty(2 * src.size, dtype=np.uint8)
    out[0::2] = src & 0xF
    out[1::2] = src >> 4
    return out


def _normalise(count: np.ndarray) -> np.ndarray:
    total = int(count.sum())
    n = count.size
    freq = np.zeros(n, dtype=np.int64)
    if total == 0:
        freq[0] = PROB_SCALE
        return freq
    largest = 0
    for s in range(n):
        c = int(count[s])
        if c == 0:
            continue
        f = c * PROB_SCALE // total
        freq[s] = 1 if f == 0 else f
        if c > int(count[largest]) or int(count[largest]) == 0:
            largest = s
    total_f = int(freq.sum())
    while total_f != PROB_SCALE:
        if total_f < PROB_SCALE:
            freq[largest] += PROB_SCALE - total_f
            break
        over = total_f - PROB_SCALE
        best = -1
        for s in range(n):
            if freq[s] > 1 and (best < 0 or freq[s] > freq[best]):
                best = s
        take = min(int(freq[best]) - 1, over)
        freq[best] -= take
        total_f -= take
    return freq


def _py_encode(src: np.ndarray, bits: int, cap: int) -> Optional[bytes]:
    nsym = 1 << bits
    sym = _symbols(src, bits)
    head = 10 + 2 * nsym
    if cap < head + 4:
        return None
    freq = _normalise(np.bincount(sym, minlength=nsym))
    cum = np.concatenate([[0], np.cumsum(freq)])
    out = bytearray()          # emitted back to front: reversed at the end
    x = LOW
    room = cap - head
    for s in sym[::-1].tolist():
        f = int(freq[s])
        x_max = ((LOW >> PROB_BITS) << 8) * f
        while x >= x_max:
            out.append(x & 0xFF)
            x >>= 8
            if len(out) > room:
                return None
        x = ((x // f) << PROB_BITS) + (x % f) + int(cum[s])
    if room - len(out) < 4:
        return None
    out += bytes([x & 0xFF, (x >> 8) & 0xFF, (x >> 16) & 0xFF, (x >> 24) & 0xFF])
    payload = bytes(reversed(out))
    return (b"R" + bytes([bits]) + struct.pack("<II", src.size, len(payload))
            + np.asarray(freq, dtype="<u2").tobytes() + payload)


def _py_decode(blob: bytes) -> bytes:
    if len(blob) < 10 or blob[0:1] != b"R" or blob[1] not in (4, 8):
        raise ValueError("rans: bad magic")
    bits = blob[1]
    nsym = 1 << bits
    nb, pb = struct.unpack_from("<II", blob, 2)
    head = 10 + 2 * nsym
    if len(blob) < head + pb or pb < 4:
        raise ValueError("rans: truncated stream")
    freq = np.frombuffer(blob, dtype="<u2", count=nsym, offset=10).astype(np.int64)
    cum = np.concatenate([[0], np.cumsum(freq)])
    if int(cum[-1]) != PROB_SCALE:
        raise ValueError("rans: bad frequency table")
    slot2sym = np.repeat(np.arange(nsym), freq)
    p = head
    end = head + pb
    x = int.from_bytes(blob[p:p + 4], "big")
    p += 4
    n = nb if bits == 8 else 2 * nb
    sym = np.empty(n, dtype=np.uint8)
    for i in range(n):
        slot = x & (PROB_SCALE - 1)
        s = int(slot2sym[slot])
        sym[i] = s
        x = int(freq[s]) * (x >> PROB_BITS) + slot - int(cum[s])
        while x < LOW:
            if p == end:
                raise ValueError("rans: truncated stream")
            x = (x << 8) | blob[p]
            p += 1
    if bits == 8:
        return sym.tobytes()
    return (sym[0::2] | (sym[1::2] << 4)).astype(np.uint8).tobytes()


# ---------------------------------------------------------------------------------------------- public coder
def rans_encode(data, bits: int = 8, budget: Optional[int] = None) -> Optional[bytes]:
    """Entropy-codes `data` (bytes / uint8 array / tensor).  `budget` is the largest accepted coded size in bytes;
    None is returned when the coded form would be larger (the caller then keeps the raw bytes)."""
    if bits not in (4, 8):
        raise ValueError("rans: 4-bit or 8-bit symbols")
    src = _as_u8(data)
    cap = rans_bound(src.size, bits) if budget is None else int(budget)
    if _LIB is None:
        return _py_encode(src, bits, cap)
    dst = np.empty(max(cap, 1), dtype=np.uint8)
    u8p = ctypes.POINTER(ctypes.c_uint8)
    keep = np.ascontiguousarray(src) if src.size else np.zeros(1, dtype=np.uint8)
    n = _LIB.nfb200_rans_encode(keep.ctypes.data_as(u8p), src.size, bits, dst.ctypes.data_as(u8p), cap)
    if n == -2:
        return None
    if n < 0:
        raise ValueError(f"rans: encoder refused its arguments ({n})")
    return dst[:n].tobytes()


def rans_decode(blob: bytes) -> bytes:
    if _LIB is None:
        return _py_decode(blob)
    if len(blob) < 10 or blob[0:1] != b"R":
        raise ValueError("rans: bad magic")
    nb = struct.unpack_from("<I", blob, 2)[0]
    src = np.frombuffer(blob, dtype=np.uint8)
    dst = np.empty(max(nb, 1), dtype=np.uint8)
    u8p = ctypes.POINTER(ctypes.c_uint8)
    n = _LIB.nfb200_rans_decode(src.ctypes.data_as(u8p), src.size, dst.ctypes.data_as(u8p), nb)
    if n < 0:
        raise ValueError({-1: "rans: bad magic", -3: "rans: truncated stream", -4: "rans: bad frequency table"}.get(n, f"rans: error {n}"))
    return dst[:nb].tobytes()


# ---------------------------------------------------------------------------------------------- cold slot
def cold_slot_bytes(rows: int, dim: int) -> int:
    """16-byte header + one nibble per value + one E4M3 scale per 16 values (9232 for a 64 x 256 page plane)."""
    return SLOT_HEADER + rows * dim // 2 + rows * dim // 16


def pack_cold_slot(values: torch.Tensor) -> bytes:
    """Requantises one [rows, dim] plane (any float dtype) to the cold slot.  Lossy by construction: a page warmed
    from its slot is not bit-identical to the page that was retired."""
    v = values.detach().to("cpu", torch.float32).numpy()
    rows, dim = v.shape
    if dim % 16:
        raise ValueError("cold slot: dim must be a multiple of 16")
    g = v.reshape(rows, dim // 16, 16)
    scale_code = L.f32_to_e4m3(np.abs(g).max(-1) / 6.0)                       # E4M3 group scale, amax -> 6
    scale = L.e4m3_to_f32(scale_code)
    inv = np.where(scale > 0, 1.0 / np.where(scale > 0, scale, 1.0), 0.0).astype(np.float32)
    codes = L.f32_to_e2m1_codes(g * inv[..., None]).reshape(rows, dim).astype(np.uint8)
    nib = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    head = struct.pack("<IHHII", SLOT_MAGIC, rows, dim, 0, 0)
    return head + nib.tobytes() + scale_code.astype(np.uint8).tobytes()


_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def restore_cold_slot(slot: bytes) -> torch.Tensor:
    """Represented values of a cold slot, fp32 [rows, dim]."""
    magic, rows, dim, _, _ = struct.unpack_from("<IHHII", slot, 0)
    if magic != SLOT_MAGIC or len(slot) != cold_slot_bytes(rows, dim):
        raise ValueError("cold slot: bad header or size")
    nib = np.frombuffer(slot, dtype=np.uint8, count=rows * dim // 2, offset=SLOT_HEADER).reshape(rows, dim // 2)
    sc = np.frombuffer(slot, dtype=np.uint8, count=rows * dim // 16, offset=SLOT_HEADER + rows * dim // 2)
    codes = np.empty((rows, dim), dtype=np.uint8)
    codes[:, 0::2] = nib & 0xF
    codes[:, 1::2] = nib >> 4
    mag = _E2M1[codes & 7] * np.where(codes & 8, -1.0, 1.0).astype(np.float32)
    scale = L.e4m3_to_f32(sc).reshape(rows, dim // 16)
    return torch.from_numpy((mag.reshape(rows, dim // 16, 16) * scale[..., None]).reshape(rows, dim).astype(np.float32))


def requant_int8_g64(codes: torch.Tensor, scales: torch.Tensor) -> bytes:
    """int8 group-64 plane (codes [rows, dim] int8, scales [rows, dim / 64] fp16) -> cold slot."""
    rows, dim = codes.shape
    v = codes.to(torch.float32).reshape(rows, dim // 64, 64) * scales.to(torch.float32)[..., None]
    return pack_cold_slot(v.reshape(rows, dim))


def restore_int8_g64(slot: bytes) -> Tuple[torch.Tensor, torch.Tensor]:
    """Cold slot -> the int8 tier's native planes (scale = fp16(amax / 127), codes clamped to +-127)."""
    v = restore_cold_slot(slot)
    rows, dim = v.shape
    g = v.reshape(rows, dim // 64, 64)
    scale = (g.abs().amax(-1) / 127.0).to(torch.float16)
    s32 = scale.to(torch.float32)
    inv = torch.where(s32 > 0, 1.0 / torch.where(s32 > 0, s32, torch.ones_like(s32)), torch.zeros_like(s32))
    codes = torch.clamp(torch.round(g * inv[..., None]), -127, 127).to(torch.int8).reshape(rows, dim)
    return codes, scale


def code_cold_slot(slot: bytes, budget_fraction: float = 0.95) -> Tuple[bytes, bool]:
    """Entropy stage of a slot: the nibble plane as 4-bit symbols and the scale plane as bytes, each kept raw when its
    coded form is not under `budget_fraction` of the raw size.  Returns (stream, any_part_coded)."""
    magic, rows, dim, _, _ = struct.unpack_from("<IHHII", slot, 0)
    n_nib = rows * dim // 2
    parts = [(slot[SLOT_HEADER:SLOT_HEADER + n_nib], 4), (slot[SLOT_HEADER + n_nib:], 8)]
    out = bytearray(slot[:SLOT_HEADER])
    coded_any = False
    for raw, bits in parts:
        blob = rans_encode(raw, bits, budget=int(len(raw) * budget_fraction)) if len(raw) else None
        if blob is None:
            out += struct.pack("<BI", 0, len(raw)) + raw
        else:
            coded_any = True
            out += struct.pack("<BI", 1, len(blob)) + blob
    return bytes(out), coded_any


def decode_cold_slot(stream: bytes) -> bytes:
    out = bytearray(stream[:SLOT_HEADER])
    p = SLOT_HEADER
    for _ in range(2):
        kind, n = struct.unpack_from("<BI", stream, p)
        p += 5
        body = stream[p:p + n]
        if len(body) != n:
            raise ValueError("cold slot stream: truncated")
        p += n
        out += rans_decode(body) if kind == 1 else body
    return bytes(out)


# ---------------------------------------------------------------------------------------------- disk tier file
FILE_MAGIC = b"NFBCOLD1"


def save_cold(cold: Dict, path: str, entropy: bool = True, budget_fraction: float = 0.97) -> Dict[str, int]:
    """Writes a demoted frontier ({"n_pages": int, "tensors": [[tensor, ...], ...]}) to `path`.  Every tensor is stored
    as raw bytes or, when that is smaller than `budget_fraction` of them, as a rANS stream (lossless).  Returns the
    byte counts {"raw", "stored", "coded_tensors"}."""
    stats = {"raw": 0, "stored": 0, "coded_tensors": 0}
    buf = io.BytesIO()
    groups = cold["tensors"]
    buf.write(FILE_MAGIC + struct.pack("<II", int(cold["n_pages"]), len(groups)))
    for group in groups:
        buf.write(struct.pack("<I", len(group)))
        for t in group:
            t = t.detach().cpu().contiguous()
            raw = t.view(torch.uint8).reshape(-1).numpy()
            blob = rans_encode(raw, 8, budget=int(raw.size * budget_fraction)) if entropy and raw.size >= 1024 else None
            dt = str(t.dtype).replace("torch.", "").encode()
            buf.write(struct.pack("<B", len(dt)) + dt + struct.pack("<B", t.dim()) + struct.pack(f"<{t.dim()}q", *t.shape))
            body = blob if blob is not None else raw.tobytes()
            buf.write(struct.pack("<BQ", 1 if blob is not None else 0, len(body)))
            buf.write(body)
            stats["raw"] += raw.size
            stats["stored"] += len(body)
            stats["coded_tensors"] += int(blob is not None)
    with open(path, "wb") as f:
        f.write(buf.getvalue())
    return stats


def load_cold(path: str) -> Dict:
    with open(path, "rb") as f:
        data = f.read()
    if data[:8] != FILE_MAGIC:
        raise ValueError(f"{path}: not a cold frontier file")
    n_pages, n_groups = struct.unpack_from("<II", data, 8)
    p = 16
    groups: List[List[torch.Tensor]] = []
    for _ in range(n_groups):
        (count,) = struct.unpack_from("<I", data, p)
        p += 4
        group = []
        for _ in range(count):
            ln = data[p]; p += 1
            dt = getattr(torch, data[p:p + ln].decode()); p += ln
            nd = data[p]; p += 1
            shape = struct.unpack_from(f"<{nd}q", data, p); p += 8 * nd
            coded, n = struct.unpack_from("<BQ", data, p); p += 9
            body = data[p:p + n]; p += n
            if len(body) != n:
                raise ValueError(f"{path}: truncated")
            raw = rans_decode(body) if coded else body
            t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dt).reshape(shape) if len(raw) else torch.empty(shape, dtype=dt)
            group.append(t)
        groups.append(group)
    return {"n_pages": n_pages, "tensors": groups}
