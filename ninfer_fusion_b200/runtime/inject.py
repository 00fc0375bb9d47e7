"""The tensor ingress: how rows chosen by the caller become context.

Every other input channel is a token channel (text) or decodes to an image (media).  This one accepts rows of the
input-embedding space directly: at declared prompt columns the row the embedding gather would have written is replaced
by the caller's row, before the first layer's norm.  After the write nothing in the forward pass can tell an injected
column from a gathered one, so

* the consumption point is the input-embedding matrix and no later tensor;
* the alphabet is the embedding space: a payload whose rows are `embed(t)` for tokens the engine could have gathered
  itself (bf16, scale 1) reproduces the plain prompt bit for bit -- the round trip is an equality, not a tolerance;
* it rides the mechanism multimodal prompts already use (rows over pad columns), so programs need no second path.

A payload is `{"dtype": "bf16" | "f16" | "f32", "scale": s, "columns": [...], "data": base64}` with `len(columns)` rows
of `hidden` elements, row-major, little endian.  It is refused, never repaired: columns must be strictly ascending and
inside the prompt, the byte count must match exactly, every element must be finite, the scale finite and non-zero, and
the result must be representable (no overflow to infinity after scaling).  bf16 with scale 1 performs no arithmetic.

Reference: src/spec/inject_channel.h (the ingress surface: consumption point, alphabet, exact round trip, refusals).
"""
from __future__ import annotations

import base64
import math
from dataclasses import dataclass, field
from typing import List, Sequence

import numpy as np
import torch

DTYPES = {"bf16": 2, "f16": 2, "f32": 4}
MAX_INJECT_ROWS = 65536


class InjectRefused(ValueError):
    pass


def decode_rows(dtype: str, data: bytes, n_rows: int, hidden: int, scale: float = 1.0) -> torch.Tensor:
    """bf16 [n_rows, hidden] from the wire bytes."""
    if dtype not in DTYPES:
        raise InjectRefused(f"dtype must be one of {sorted(DTYPES)}")
    if not isinstance(scale, (int, float)) or isinstance(scale, bool) or not math.isfinite(scale) or scale == 0:
        raise InjectRefused("scale must be a finite non-zero number")
    want = n_rows * hidden * DTYPES[dtype]
    if len(data) != want:
        raise InjectRefused(f"payload has {len(data)} bytes; {n_rows} rows of {hidden} {dtype} elements take {want}")
    if dtype == "bf16":
        words = np.frombuffer(data, dtype="<u2").astype(np.int16).reshape(n_rows, hidden)
        rows = torch.from_numpy(words.copy()).view(torch.bfloat16)
        if not torch.isfinite(rows.float()).all():
            raise InjectRefused("payload holds a NaN or an infinity")
        if scale == 1:
            return rows                       # the identity: the same 16-bit words, no arithmetic
        out = rows.float() * float(scale)
    else:
        arr = np.frombuffer(data, dtype="<f2" if dtype == "f16" else "<f4").reshape(n_rows, hidden)
        out = torch.from_numpy(arr.astype(np.float32)) * float(scale)
        if not np.isfinite(arr).all():
            raise InjectRefused("payload holds a NaN or an infinity")
    out = out.to(torch.bfloat16)
    if not torch.isfinite(out.float()).all():
        raise InjectRefused("scaled payload overflows bf16")
    return out


def encode_rows(rows: torch.Tensor, dtype: str = "bf16") -> bytes:
    """Wire bytes of rows (the inverse of `decode_rows` at scale 1)."""
    if dtype == "bf16":
        return rows.to(torch.bfloat16).contiguous().view(torch.int16).numpy().astype("<i2").tobytes()
    return rows.float().numpy().astype("<f2" if dtype == "f16" else "<f4").tobytes()


@dataclass
class InjectedPrompt:
    """A prompt with injected rows, in the shape programs already consume multimodal prompts in: plain sequential
    positions on all three rotary axes, no media items, `embed_rows` = the columns, `rows` = what goes there."""
    ids: List[int]
    positions: np.ndarray
    rope_delta: int
    embed_rows: np.ndarray
    rows: torch.Tensor
    items: list = field(default_factory=list)

    @property
    def grids(self):
        return []

    def patches(self):
        return torch.zeros((0, 0), dtype=torch.bfloat16)


def build_injected_prompt(ids: Sequence[int], columns: Sequence[int], rows: torch.Tensor, hidden: int) -> InjectedPrompt:
    cols = [int(c) for c in columns]
    if not cols:
        raise InjectRefused("no columns")
    if len(cols) > MAX_INJECT_ROWS:
        raise InjectRefused(f"at most {MAX_INJECT_ROWS} rows per request")
    if any(b <= a for a, b in zip(cols, cols[1:])):
        raise InjectRefused("columns must be strictly ascending")
    if cols[0] < 0 or cols[-1] >= len(ids):
        raise InjectRefused(f"columns must lie inside the prompt (0..{len(ids) - 1})")
    if tuple(rows.shape) != (len(cols), hidden) or rows.dtype != torch.bfloat16:
        raise InjectRefused(f"rows must be bf16 [{len(cols)}, {hidden}]")
    t = np.arange(len(ids), dtype=np.int32)
    return InjectedPrompt(list(int(i) for i in ids), np.stack([t, t, t], axis=1), 0, np.asarray(cols, dtype=np.int32),
                          rows.contiguous())


def parse_injection(payload: dict, ids: Sequence[int], hidden: int) -> InjectedPrompt:
    if not isinstance(payload, dict):
        raise InjectRefused("the injection is an object")
    unknown = set(payload) - {"dtype", "scale", "columns", "data"}
    if unknown:
        raise InjectRefused(f"unknown fields: {sorted(unknown)}")
    cols = payload.get("columns")
    if not isinstance(cols, list) or not all(isinstance(c, int) and not isinstance(c, bool) for c in cols):
        raise InjectRefused("columns is a list of integers")
    try:
        data = base64.b64decode(payload.get("data", ""), validate=True)
    except (ValueError, TypeError):
        raise InjectRefused("data is not base64") from None
    rows = decode_rows(str(payload.get("dtype", "bf16")), data, len(cols), hidden, payload.get("scale", 1.0))
    return build_injected_prompt(ids, cols, rows, hidden)
