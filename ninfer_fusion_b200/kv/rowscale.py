"""K row-scale loop: solve, persist, validate and load the per-channel multipliers of the stored K frame.

For every full-attention (layer, kv_head) a per-channel ``s_d`` in [0.5, 2] balances the channel RMS of K before it is
quantised; K is multiplied by ``s_d`` when it is written to the cache and Q by ``1 / s_d`` before Q.K, so the scores
are unchanged while low-bit codecs (nvfp4 groups of 16, fp8 rows) stop spending their range on a few loud channels.

* ``solve_row_scale``: the constrained balancing iteration on sampled K rows (the reference's Sinkhorn row scale,
  src/ops/kernel/gqa_isoquant_row_scale.cuh; tools/calib).
* ``write_table`` / ``read_table`` / ``validate``: the side file ``<artifact>.kvrowscale.bin`` -- 64-byte header
  ``NINFERKVRS1`` + BF16 ``[layer][kv_head][d]`` with CRC and model hash, and the identity rules of the reference's
  parser (tools/kv_rowscale_sidecar.py:12-40, src/product/kv_rowscale_persist.h:25-40).
* ``load_into``: hands the per-layer tables to a device model (``HybridModel.k_row_scale``) or to oracle sequences.
"""
from __future__ import annotations

import struct
import zlib
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import torch

MAGIC = b"NINFERKVRS1"
HEADER_BYTES = 64
VERSION = 1
FLAG_IDENTITY = 1
S_MIN, S_MAX = 0.5, 2.0
SIDE_SUFFIX = ".kvrowscale.bin"


class RowScaleError(ValueError):
    pass


def solve_row_scale(k_rows: torch.Tensor, iters: int = 16) -> torch.Tensor:
    """k_rows: [n, D] samples of one (layer, kv_head) in the frame K is stored in.  Returns s: [D] in [0.5, 2].

    Unconstrained, s_d = target / rms_d equalises every channel.  The clamp to [0.5, 2] breaks that for loud or silent
    channels, so the target is re-fitted to the channels that are still free (geometric mean of their RMS, which keeps
    the product of the free multipliers at one) until the clamped set stops changing."""
    x = k_rows.detach().to(torch.float32)
    rms = x.pow(2).mean(0).sqrt().clamp_min(1e-12)
    log_rms = rms.log()
    free = torch.ones_like(rms, dtype=torch.bool)
    s = torch.ones_like(rms)
    for _ in range(max(1, iters)):
        target = log_rms[free].mean() if free.any() else log_rms.mean()
        s = (target - log_rms).exp().clamp(S_MIN, S_MAX)
        now_free = (s > S_MIN) & (s < S_MAX)
        if torch.equal(now_free, free):
            break
        free = now_free
    # the table is stored as bf16: return exactly what will be applied
    return s.to(torch.bfloat16).to(torch.float32)


def balance_gain(k_rows: torch.Tensor, s: torch.Tensor) -> float:
    """max / min channel RMS before, divided by the same after scaling (> 1 means the rows got flatter)."""
    x = k_rows.detach().to(torch.float32)
    r0 = x.pow(2).mean(0).sqrt().clamp_min(1e-12)
    r1 = (x * s).pow(2).mean(0).sqrt().clamp_min(1e-12)
    return float((r0.max() / r0.min()) / (r1.max() / r1.min()))


@dataclass
class RowScaleTable:
    scales: torch.Tensor          # [layers, kv_heads, head_dim] bf16
    identity: bool = False
    model_hash: int = 0
    tag: str = ""

    @property
    def geometry(self):
        return tuple(self.scales.shape)


def write_table(path: str, scales: torch.Tensor, tag: str = "", model_hash: int = 0, identity: Optional[bool] = None) -> None:
    if scales.dim() != 3:
        raise RowScaleError("row-scale table must be [layers, kv_heads, head_dim]")
    t = scales.detach().to("cpu", torch.bfloat16).contiguous()
    f32 = t.to(torch.float32)
    is_identity = bool((f32 == 1.0).all())
    if identity is None:
        identity = is_identity
    if identity and not is_identity:
        raise RowScaleError("identity flag set but a word is not BF16 1.0")
    if not identity and (f32.min() < S_MIN or f32.max() > S_MAX):
        raise RowScaleError(f"row scales must lie in [{S_MIN}, {S_MAX}]")
    payload = t.view(torch.int16).numpy().tobytes()
    tag_b = tag.encode("utf-8")
    if len(tag_b) > 16:
        raise RowScaleError("tag is longer than 16 bytes")
    L, H, D = t.shape
    head = (MAGIC.ljust(16, b"\0") + struct.pack("<IIIIII", VERSION, L, H, D, FLAG_IDENTITY if identity else 0,
                                                 zlib.crc32(payload) & 0xFFFFFFFF)
            + struct.pack("<Q", model_hash & 0xFFFFFFFFFFFFFFFF) + tag_b.ljust(16, b"\0"))
    assert len(head) == HEADER_BYTES
    with open(path, "wb") as f:
        f.write(head + payload)


def read_table(path: str) -> RowScaleTable:
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < HEADER_BYTES:
        raise RowScaleError("file is shorter than its header")
    if data[:11] != MAGIC or any(data[11:16]):
        raise RowScaleError("magic: not a NINFERKVRS1 table")
    version, L, H, D, flags, crc = struct.unpack_from("<IIIIII", data, 16)
    (model_hash,) = struct.unpack_from("<Q", data, 40)
    tag = data[48:64].rstrip(b"\0").decode("utf-8", "replace")
    if version != VERSION:
        raise RowScaleError(f"version: {version} is not {VERSION}")
    if flags & ~FLAG_IDENTITY:
        raise RowScaleError(f"flags: unknown bits {flags:#x}")
    payload = data[HEADER_BYTES:]
    if len(payload) != 2 * L * H * D:
        raise RowScaleError(f"payload: {len(payload)} bytes, geometry {L} x {H} x {D} needs {2 * L * H * D}")
    if zlib.crc32(payload) & 0xFFFFFFFF != crc:
        raise RowScaleError("crc32: payload does not match the header")
    t = torch.frombuffer(bytearray(payload), dtype=torch.int16).view(torch.bfloat16).reshape(L, H, D).clone()
    identity = bool(flags & FLAG_IDENTITY)
    f32 = t.to(torch.float32)
    if identity and not bool((f32 == 1.0).all()):
        raise RowScaleError("flags: identity table with a word that is not BF16 1.0")
    if not identity and (not torch.isfinite(f32).all() or f32.min() < S_MIN or f32.max() > S_MAX):
        raise RowScaleError(f"payload: a scale lies outside [{S_MIN}, {S_MAX}]")
    return RowScaleTable(t, identity, model_hash, tag)


def validate(table: RowScaleTable, layers: int, kv_heads: int, head_dim: int, model_hash: int = 0) -> None:
    """Geometry rules of the loader: a real table must match the model exactly (a 16-layer table under a 52-layer
    model is refused); an identity table may cover fewer layers.  A non-zero model hash on both sides must agree."""
    L, H, D = table.geometry
    if H != kv_heads:
        raise RowScaleError(f"kv_heads: table has {H}, model has {kv_heads}")
    if D != head_dim:
        raise RowScaleError(f"head_dim: table has {D}, model has {head_dim}")
    if table.identity:
        if L > layers:
            raise RowScaleError(f"layers: identity table covers {L} layers, model has {layers}")
    elif L != layers:
        raise RowScaleError(f"layers: table has {L}, model has {layers}")
    if model_hash and table.model_hash and model_hash != table.model_hash:
        raise RowScaleError(f"model_hash: table {table.model_hash:#x}, model {model_hash:#x}")


def load_into(model, table: RowScaleTable, attn_layers: Sequence[int], kv_head_slice: Optional[slice] = None) -> int:
    """Gives `model` (anything with a ``k_row_scale`` dict and a ``device``) the table rows of its attention layers.
    The table is indexed by attention-layer ordinal; the model's dict by absolute layer index.  A tensor-parallel
    shard passes the slice of kv heads it owns.  Identity tables load nothing.  Returns the number of layers set."""
    if table.identity:
        return 0
    n = 0
    for ordinal, layer in enumerate(attn_layers):
        if ordinal >= table.scales.shape[0]:
            break
        rows = table.scales[ordinal]
        if kv_head_slice is not None:
            rows = rows[kv_head_slice]
        model.k_row_scale[layer] = rows.contiguous().to(getattr(model, "device", "cpu"))
        n += 1
    return n


def side_file(artifact_path: str) -> str:
    return artifact_path + SIDE_SUFFIX
