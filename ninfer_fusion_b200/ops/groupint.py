"""Groupwise-integer weights (Q4/Q5/Q6 with 64-value groups, W8 with 32-value groups) used without re-encoding.

``GroupIntWeight`` keeps the artifact's encoded row-split object (nibble plane, high-bit plane, fp16 group scales) on
the device; ``linear`` / ``linear_pair`` stream it through ``torch.ops.nfb200.groupint_linear*`` (in-register dequant,
``mma.sync``, at most 32 tokens per weight pass).  Counterparts in the reference: the q4 / q5 / q6 / w8 row-split
kernels under ``src/ops/linear``, ``src/ops/linear_add`` and ``src/ops/linear_pair/w8``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..artifact import layouts as L

FORMAT_IDS = {"Q4G64_F16S": 0, "Q5G64_F16S": 1, "Q6G64_F16S": 2, "W8G32_F16S": 3}
SHORT_NAMES = {"q4": "Q4G64_F16S", "q5": "Q5G64_F16S", "q6": "Q6G64_F16S", "w8": "W8G32_F16S"}
QT_GROUPINT = 3   # qtype tag beside ops.quant.QT_FP8_ROW (1) and QT_NVFP4 (2)


class GroupIntWeight:
    """One [N, K] matmul weight as an encoded row-split object on the device."""
    __slots__ = ("fmt", "payload", "shape", "qtype", "_dense", "rot_block")

    def __init__(self, fmt: str, payload: torch.Tensor, shape, rot_block: int = 0):
        if fmt not in FORMAT_IDS:
            raise ValueError(f"not a groupwise-int format: {fmt}")
        N, K = (int(s) for s in shape)
        need = L.encoded_size(fmt, "row-split-k128-v1", (N, K))
        if payload.dtype != torch.uint8 or payload.numel() < need:
            raise ValueError(f"payload of {payload.numel()} bytes cannot hold a {fmt} [{N}, {K}] object ({need} bytes)")
        self.fmt, self.payload, self.shape, self.qtype, self._dense = fmt, payload, (N, K), QT_GROUPINT, None
        # > 0: the codes hold W H (input dimension rotated block-wise, ops/rotation.py); consumers rotate x the same way
        self.rot_block = int(rot_block)

    @classmethod
    def from_dense(cls, w: torch.Tensor, fmt: str, device=None, rot_block: int = 0) -> "GroupIntWeight":
        fmt = SHORT_NAMES.get(fmt, fmt)
        dev = device if device is not None else w.device
        if rot_block:
            from .rotation import fold
            w = fold(w.detach().to("cpu", torch.float32), rot_block)
        w32 = w.detach().to("cpu", torch.float32).numpy()
        codes, scale = L.quantize_group_int(w32, fmt)
        raw = L.encode_row_split(codes, scale, fmt, w32.shape[1])
        payload = torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).copy())
        return cls(fmt, payload.to(dev), w.shape, rot_block)

    @property
    def fmt_id(self) -> int:
        return FORMAT_IDS[self.fmt]

    def nbytes(self) -> int:
        return self.payload.numel()

    def usable_by_kernel(self) -> bool:
        N, K = self.shape
        return N % 16 == 0 and K % 64 == 0

    def dequant_stored(self) -> torch.Tensor:
        """Values of the stored codes, fp32 [N, K] on the CPU (W H when the weight is rotated)."""
        raw = self.payload.cpu().numpy().tobytes()
        codes, scale = L.decode_row_split(raw, self.fmt, self.shape)
        return torch.from_numpy(L.dequant_row_split(codes, scale, self.fmt, self.shape[1]).astype(np.float32))

    def dequant(self) -> torch.Tensor:
        """Represented weight, fp32 [N, K] on the CPU (the oracle's weight): a rotated weight is rotated back,
        H being its own inverse."""
        w = self.dequant_stored()
        if self.rot_block:
            from .rotation import fold
            w = fold(w, self.rot_block)
        return w

    def dense(self) -> torch.Tensor:
        """bf16 copy on the device for token counts the streaming kernel is not meant for (made once, kept)."""
        if self._dense is None:
            self._dense = self.dequant().to(self.payload.device, torch.bfloat16)
        return self._dense


def linear(ops, x: torch.Tensor, w: GroupIntWeight, out: Optional[torch.Tensor] = None,
           resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x @ w^T (+ resid); x bf16 [T, K].  Any T is accepted; the weights are read once per 32 tokens."""
    N, K = w.shape
    if out is None:
        out = torch.empty((x.shape[0], N), dtype=torch.bfloat16, device=x.device)
    if w.rot_block:
        from .rotation import rotate
        x = rotate(ops, x, w.rot_block)
    ops.groupint_linear(x, w.payload, w.fmt_id, N, K, out, resid)
    return out


def linear_pair(ops, x: torch.Tensor, w0: GroupIntWeight, w1: GroupIntWeight) -> Tuple[torch.Tensor, torch.Tensor]:
    """Two projections of one input in one launch (the reference's linear_pair: MTP K / V projections)."""
    if w0.fmt != w1.fmt or w0.shape[1] != w1.shape[1]:
        raise ValueError("linear_pair: both weights must share the format and the input width")
    if w0.rot_block != w1.rot_block:
        raise ValueError("linear_pair: both weights must share the input rotation")
    if w0.rot_block:
        from .rotation import rotate
        x = rotate(ops, x, w0.rot_block)
    T = x.shape[0]
    o0 = torch.empty((T, w0.shape[0]), dtype=torch.bfloat16, device=x.device)
    o1 = torch.empty((T, w1.shape[0]), dtype=torch.bfloat16, device=x.device)
    ops.groupint_linear_pair(x, w0.payload, w0.shape[0], w1.payload, w1.shape[0], w0.fmt_id, w0.shape[1], o0, o1)
    return o0, o1


def linear_reference(x: torch.Tensor, w: GroupIntWeight, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 oracle on the CPU: bf16 activations as given, represented weight values, exact sums."""
    y = x.detach().to("cpu", torch.float32) @ w.dequant().t()
    if resid is not None:
        y = y + resid.detach().to("cpu", torch.float32)
    return y
