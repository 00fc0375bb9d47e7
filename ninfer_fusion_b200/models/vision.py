"""Vision tower: patch rows -> merged visual tokens in the text model's hidden width.

Schedule (src/targets/qwen3_6/impl/runtime/vision_context_impl.h:300-387, math in
docs/maintainer/qwen3.6-27b-model.md section 10): patch projection + bias, bilinear position table,
27 x {LayerNorm, qkv + bias, 2-D rope, packed bidirectional attention, projection + bias + residual,
LayerNorm, fc1 + bias + GELU(tanh), fc2 + bias + residual}, merger {LayerNorm, 2x2 merge, fc1 + bias +
GELU(erf), fc2 + bias}.

The reference launches bias / GELU / residual as separate pointwise ops; here they are epilogues of the
tcgen05 GEMM (`gemm_bf16` with bias, activation, residual), so a block is 8 launches: 2 LayerNorm,
4 GEMM, rope, attention.  Position-table corners and weights are computed inside the kernel from the
patch's grid coordinates instead of being uploaded.

`vision_reference` is the plain PyTorch fp32 oracle of the same math (bf16 rounding at the points where
the device path stores bf16).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

EPI_STORE, EPI_RESIDUAL = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2


@dataclass(frozen=True)
class VisionConfig:
    """Geometry of the tower (src/targets/qwen3_6/export/ninfer/targets/qwen3_6/vision.h:15-29)."""
    layers: int = 27
    hidden: int = 1152
    intermediate: int = 4304
    heads: int = 16
    patch: int = 16
    temporal: int = 2
    channels: int = 3
    merge: int = 2
    pos_side: int = 48
    out_hidden: int = 5120
    rope_theta: float = 10000.0
    eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def patch_dim(self) -> int:
        return self.channels * self.temporal * self.patch * self.patch

    @property
    def merge_unit(self) -> int:
        return self.merge * self.merge

    @property
    def merger_hidden(self) -> int:
        return self.hidden * self.merge_unit

    def scaled(self, layers: int, out_hidden: int) -> "VisionConfig":
        """Same geometry with fewer blocks / another text width (tests, small packages)."""
        return VisionConfig(layers, self.hidden, self.intermediate, self.heads, self.patch, self.temporal,
                            self.channels, self.merge, self.pos_side, out_hidden, self.rope_theta, self.eps)


def vision_leaves(cfg: VisionConfig) -> Dict[str, Tuple[int, ...]]:
    """Name -> shape of every tensor of the tower (matrices are [out, in])."""
    H, I = cfg.hidden, cfg.intermediate
    out: Dict[str, Tuple[int, ...]] = {
        "vision/patch_embed": (H, cfg.patch_dim), "vision/patch_embed_bias": (H,),
        "vision/pos_embed": (cfg.pos_side * cfg.pos_side, H),
        "vision/merger/norm_w": (H,), "vision/merger/norm_b": (H,),
        "vision/merger/fc1": (cfg.merger_hidden, cfg.merger_hidden), "vision/merger/fc1_bias": (cfg.merger_hidden,),
        "vision/merger/fc2": (cfg.out_hidden, cfg.merger_hidden), "vision/merger/fc2_bias": (cfg.out_hidden,),
    }
    for l in range(cfg.layers):
        p = f"vision/blocks/{l}"
        out.update({f"{p}/norm1_w": (H,), f"{p}/norm1_b": (H,), f"{p}/qkv": (3 * H, H), f"{p}/qkv_bias": (3 * H,),
                    f"{p}/proj": (H, H), f"{p}/proj_bias": (H,), f"{p}/norm2_w": (H,), f"{p}/norm2_b": (H,),
                    f"{p}/fc1": (I, H), f"{p}/fc1_bias": (I,), f"{p}/fc2": (H, I), f"{p}/fc2_bias": (H,)})
    return out


def random_vision_weights(cfg: VisionConfig, device="cpu", seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init tower in bf16 (norm weights around 1, small biases)."""
    g = torch.Generator().manual_seed(seed)
    w: Dict[str, torch.Tensor] = {}
    for name, shape in vision_leaves(cfg).items():
        if name.endswith("norm_w") or name.endswith("norm1_w") or name.endswith("norm2_w"):
            t = 1.0 + 0.05 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.02 * torch.randn(shape, generator=g)
        elif name.endswith("pos_embed"):
            t = 0.05 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        w[name] = t.to(torch.bfloat16).to(device)
    return w


# ---------------------------------------------------------------------------------------- control
@dataclass
class VisionControl:
    """Per-patch metadata of one encode call (src/targets/qwen3_6/impl/vision/control.cpp:111-200)."""
    pos_yx: np.ndarray     # int32 [P, 2] patch row / column inside its frame grid
    grid_hw: np.ndarray    # int32 [P, 2] the grid's height / width
    segments: np.ndarray   # int32 [S + 1] cumulative patch counts: one attention segment per frame
    n_patches: int
    n_tokens: int          # merged tokens (P / merge^2)


def build_control(grids: Sequence[Tuple[int, int, int]], merge: int = 2) -> VisionControl:
    """`grids` = (temporal, height, width) in patches per media item.  Patches are ordered frame by frame, inside a
    frame merge-block by merge-block (so the merger's 2x2 group is four consecutive rows)."""
    pos, ghw, seg = [], [], [0]
    for (t, h, w) in grids:
        if h % merge or w % merge or t < 1:
            raise ValueError(f"grid {(t, h, w)} is not a multiple of the merge size {merge}")
        by, bx, iy, ix = np.meshgrid(np.arange(h // merge), np.arange(w // merge), np.arange(merge), np.arange(merge),
                                     indexing="ij")
        y = (by * merge + iy).reshape(-1)
        x = (bx * merge + ix).reshape(-1)
        frame = np.stack([y, x], axis=1).astype(np.int32)
        for _ in range(t):
            pos.append(frame)
            ghw.append(np.tile(np.array([[h, w]], dtype=np.int32), (h * w, 1)))
            seg.append(seg[-1] + h * w)
    P = seg[-1]
    return VisionControl(np.concatenate(pos) if pos else np.zeros((0, 2), np.int32),
                         np.concatenate(ghw) if ghw else np.zeros((0, 2), np.int32),
                         np.array(seg, dtype=np.int32), P, P // (merge * merge))


def attention_tiles(segments: np.ndarray, tile: int) -> np.ndarray:
    """[n, 3] rows (first query row, segment begin, segment end): `tile` queries per row."""
    rows = []
    for s in range(len(segments) - 1):
        b, e = int(segments[s]), int(segments[s + 1])
        rows.extend((q, b, e) for q in range(b, e, tile))
    return np.array(rows, dtype=np.int32).reshape(-1, 3)


# ---------------------------------------------------------------------------------------- device path
class VisionTower:
    """Runs the tower on the native kernels; buffers grow to the largest request seen."""

    def __init__(self, cfg: VisionConfig, weights: Dict[str, torch.Tensor], device):
        from .._lib import load_native
        from .hybrid import LaunchCounter
        self.cfg = cfg
        self.device = torch.device(device)
        self.ops = LaunchCounter(load_native())
        self.w = {k: v.to(self.device) for k, v in weights.items() if k.startswith("vision/")}
        missing = [k for k in vision_leaves(cfg) if k not in self.w]
        if missing:
            raise KeyError(f"vision weights missing: {missing[:4]}{'...' if len(missing) > 4 else ''}")
        # GEMM biases are read as fp32 by the epilogue
        self.bias = {k: v.float().contiguous() for k, v in self.w.items() if k.endswith("_bias")}
        self.tile = int(self.ops.packed_attention_tile())
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._cap = 0
        self.launches = 0

    def _reserve(self, P: int) -> None:
        if P <= self._cap:
            return
        cfg, dev, bf = self.cfg, self.device, torch.bfloat16
        cap = (P + 255) // 256 * 256
        self.x = torch.empty((cap, cfg.hidden), dtype=bf, device=dev)
        self.h = torch.empty((cap, cfg.hidden), dtype=bf, device=dev)
        self.qkv = torch.empty((cap, 3 * cfg.hidden), dtype=bf, device=dev)
        self.att = torch.empty((cap, cfg.hidden), dtype=bf, device=dev)
        self.mlp = torch.empty((cap, cfg.intermediate), dtype=bf, device=dev)
        self.merged = torch.empty((cap // cfg.merge_unit, cfg.merger_hidden), dtype=bf, device=dev)
        self._cap = cap

    def _gemm(self, x, w, out, epi=EPI_STORE, resid=None, bias=None, act=ACT_NONE):
        self.ops.gemm_bf16(x, w, out, epi, resid, bias, None, 1, self.status, False, act)

    def encode(self, patches: torch.Tensor, control: VisionControl, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """patches: bf16 [P, patch_dim] (host or device) -> bf16 [P / merge^2, out_hidden]."""
        cfg, ops, w, b = self.cfg, self.ops, self.w, self.bias
        P = control.n_patches
        if patches.shape != (P, cfg.patch_dim) or patches.dtype != torch.bfloat16:
            raise ValueError(f"patches must be bf16 [{P}, {cfg.patch_dim}]")
        if P == 0 or P % cfg.merge_unit:
            raise ValueError("patch count must be a positive multiple of the merge unit")
        self._reserve(P)
        dev = self.device
        start = ops.count
        patches = patches.to(dev, non_blocking=True)
        pos = torch.from_numpy(control.pos_yx).to(dev, non_blocking=True)
        ghw = torch.from_numpy(control.grid_hw).to(dev, non_blocking=True)
        tiles = torch.from_numpy(attention_tiles(control.segments, self.tile)).to(dev, non_blocking=True)
        x, h, qkv, att, mlp = self.x[:P], self.h[:P], self.qkv[:P], self.att[:P], self.mlp[:P]
        self._gemm(patches, w["vision/patch_embed"], x, bias=b["vision/patch_embed_bias"])
        ops.vision_pos_embed_add(x, w["vision/pos_embed"], pos, ghw, cfg.pos_side)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        for l in range(cfg.layers):
            p = f"vision/blocks/{l}"
            ops.layer_norm(x, w[f"{p}/norm1_w"], w[f"{p}/norm1_b"], h, cfg.eps)
            self._gemm(h, w[f"{p}/qkv"], qkv, bias=b[f"{p}/qkv_bias"])
            ops.vision_rope(qkv, pos, cfg.heads, cfg.head_dim, cfg.rope_theta)
            ops.packed_attention(qkv, att, tiles, cfg.heads, scale)
            self._gemm(att, w[f"{p}/proj"], x, EPI_RESIDUAL, x, b[f"{p}/proj_bias"])
            ops.layer_norm(x, w[f"{p}/norm2_w"], w[f"{p}/norm2_b"], h, cfg.eps)
            self._gemm(h, w[f"{p}/fc1"], mlp, bias=b[f"{p}/fc1_bias"], act=ACT_GELU_TANH)
            self._gemm(mlp, w[f"{p}/fc2"], x, EPI_RESIDUAL, x, b[f"{p}/fc2_bias"])
        ops.layer_norm(x, w["vision/merger/norm_w"], w["vision/merger/norm_b"], h, cfg.eps)
        V = P // cfg.merge_unit
        merged_in = h.view(V, cfg.merger_hidden)
        merged = self.merged[:V]
        self._gemm(merged_in, w["vision/merger/fc1"], merged, bias=b["vision/merger/fc1_bias"], act=ACT_GELU_ERF)
        if out is None:
            out = torch.empty((V, cfg.out_hidden), dtype=torch.bfloat16, device=dev)
        self._gemm(merged, w["vision/merger/fc2"], out, bias=b["vision/merger/fc2_bias"])
        self.launches = ops.count - start
        return out


# ---------------------------------------------------------------------------------------- oracle
def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def _lin(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return x @ w.float().t() + b.float()


def pos_embed_reference(table: torch.Tensor, control: VisionControl, side: int) -> torch.Tensor:
    """Bilinear interpolation of the [side*side, D] table at every patch (fp32)."""
    y, x = torch.from_numpy(control.pos_yx[:, 0]).float(), torch.from_numpy(control.pos_yx[:, 1]).float()
    h, w = torch.from_numpy(control.grid_hw[:, 0]).float(), torch.from_numpy(control.grid_hw[:, 1]).float()
    yf = torch.where(h > 1, y * (side - 1) / (h - 1).clamp(min=1), torch.zeros_like(y))
    xf = torch.where(w > 1, x * (side - 1) / (w - 1).clamp(min=1), torch.zeros_like(x))
    y0, x0 = yf.floor().long(), xf.floor().long()
    y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
    wy, wx = (yf - y0.float())[:, None], (xf - x0.float())[:, None]
    t = table.float()
    return (t[y0 * side + x0] * (1 - wy) * (1 - wx) + t[y0 * side + x1] * (1 - wy) * wx +
            t[y1 * side + x0] * wy * (1 - wx) + t[y1 * side + x1] * wy * wx)


def rope_2d_reference(x: torch.Tensor, pos_yx: torch.Tensor, theta: float) -> torch.Tensor:
    """x [P, H, D]: pair i = (d_i, d_{i + D/2}); pairs [0, D/4) turn with y, [D/4, D/2) with x
    (include/ninfer/ops/rope.h:63-95)."""
    D = x.shape[-1]
    half, quarter = D // 2, D // 4
    inv = theta ** (-2.0 * torch.arange(quarter).float() / half)
    ang = torch.cat([pos_yx[:, 0:1].float() * inv[None], pos_yx[:, 1:2].float() * inv[None]], dim=1)  # [P, half]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1)


def packed_attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, segments: np.ndarray,
                               scale: float) -> torch.Tensor:
    """q, k, v [P, H, D] fp32; bidirectional attention inside each segment."""
    out = torch.zeros_like(q)
    for s in range(len(segments) - 1):
        b, e = int(segments[s]), int(segments[s + 1])
        sc = torch.einsum("qhd,khd->hqk", q[b:e], k[b:e]) * scale
        out[b:e] = torch.einsum("hqk,khd->qhd", torch.softmax(sc, dim=-1), v[b:e])
    return out


def vision_reference(cfg: VisionConfig, weights: Dict[str, torch.Tensor], patches: torch.Tensor,
                     control: VisionControl) -> torch.Tensor:
    """fp32 oracle of `VisionTower.encode` on the CPU."""
    w = {k: v.detach().cpu() for k, v in weights.items() if k.startswith("vision/")}
    P, H, D = control.n_patches, cfg.heads, cfg.head_dim
    pos = torch.from_numpy(control.pos_yx)
    x = _bf(_lin(patches.float().cpu(), w["vision/patch_embed"], w["vision/patch_embed_bias"]))
    x = _bf(x + pos_embed_reference(w["vision/pos_embed"], control, cfg.pos_side))
    ln = torch.nn.functional.layer_norm
    for l in range(cfg.layers):
        p = f"vision/blocks/{l}"
        h = _bf(ln(x, (cfg.hidden,), w[f"{p}/norm1_w"].float(), w[f"{p}/norm1_b"].float(), cfg.eps))
        qkv = _bf(_lin(h, w[f"{p}/qkv"], w[f"{p}/qkv_bias"])).view(P, 3, H, D)
        q = _bf(rope_2d_reference(qkv[:, 0], pos, cfg.rope_theta))
        k = _bf(rope_2d_reference(qkv[:, 1], pos, cfg.rope_theta))
        a = _bf(packed_attention_reference(q, k, qkv[:, 2], control.segments, 1.0 / math.sqrt(D))).reshape(P, H * D)
        x = _bf(x + _lin(a, w[f"{p}/proj"], w[f"{p}/proj_bias"]))
        h = _bf(ln(x, (cfg.hidden,), w[f"{p}/norm2_w"].float(), w[f"{p}/norm2_b"].float(), cfg.eps))
        m = _bf(torch.nn.functional.gelu(_lin(h, w[f"{p}/fc1"], w[f"{p}/fc1_bias"]), approximate="tanh"))
        x = _bf(x + _lin(m, w[f"{p}/fc2"], w[f"{p}/fc2_bias"]))
    h = _bf(ln(x, (cfg.hidden,), w["vision/merger/norm_w"].float(), w["vision/merger/norm_b"].float(), cfg.eps))
    merged = h.view(P // cfg.merge_unit, cfg.merger_hidden)
    m = _bf(torch.nn.functional.gelu(_lin(merged, w["vision/merger/fc1"], w["vision/merger/fc1_bias"])))
    return _bf(_lin(m, w["vision/merger/fc2"], w["vision/merger/fc2_bias"]))
