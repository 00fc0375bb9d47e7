"""E8-lattice quantiser for K rows (oracle and tier arithmetic; no device kernel reads this tier).

E8 = D8 u (D8 + 1/2): vectors of eight integers with an even sum, or eight half-integers with an even sum.  Per point
of volume it has the lowest mean squared error of any 8-dimensional lattice (0.65 dB under the cubic lattice), which
is what the reference's rk4v4 / rk3v4 / rk2v4 tiers buy for K at 4 / 3 / 2 bits per value
(src/ops/kv_cache e8_lattice_*, rk2v4e8_codec.cuh).  A row is divided by one fp16 scale per group of 64 values and
snapped to the lattice in blocks of eight; the clamp radius fixes the code width.

* ``nearest_e8``: exact nearest lattice point (the two-coset rounding of Conway and Sloane).
* ``quant_dequant``: the tier's value map for a tensor whose last dimension is a multiple of 64.
* ``bits_per_value``: code bits + scale bits of a tier, as the bit-budget planner counts them.
"""
from __future__ import annotations

import math

import torch

GROUP = 64
TIER_RADIUS = {"rk4v4": 7.5, "rk3v4": 3.5, "rk2v4": 1.5}      # clamp of a coordinate, in lattice units


def _nearest_d8(x: torch.Tensor) -> torch.Tensor:
    """Nearest point of D8 (integers, even sum): round everything; if the sum is odd, re-round the coordinate that was
    furthest from its integer the other way."""
    r = torch.round(x)
    odd = (r.sum(-1).to(torch.int64) % 2) != 0
    err = x - r
    worst = err.abs().argmax(-1, keepdim=True)
    step = torch.where(torch.gather(err, -1, worst) >= 0, 1.0, -1.0)
    fixed = r.scatter_add(-1, worst, step)
    return torch.where(odd[..., None], fixed, r)


def nearest_e8(x: torch.Tensor) -> torch.Tensor:
    """x: [..., 8] -> nearest point of E8."""
    if x.shape[-1] != 8:
        raise ValueError("E8 works on blocks of eight values")
    x = x.to(torch.float32)
    a = _nearest_d8(x)
    b = _nearest_d8(x - 0.5) + 0.5
    da, db = (x - a).pow(2).sum(-1, keepdim=True), (x - b).pow(2).sum(-1, keepdim=True)
    return torch.where(da <= db, a, b)


def in_e8(p: torch.Tensor) -> torch.Tensor:
    twice = torch.round(2 * p)
    all_int = ((twice % 2) == 0).all(-1)
    all_half = ((twice % 2) != 0).all(-1)
    even = (torch.round(p.sum(-1)) % 2) == 0
    exact = (2 * p - twice).abs().max(-1).values < 1e-6
    return exact & (all_int | all_half) & even


def bits_per_value(tier: str) -> float:
    """K code width of the tier: log2 of the lattice points inside the clamp cube per 8 values, plus one fp16 scale per
    64.  E8 has one point per unit volume, so the cube [-R, R]^8 holds about (2R)^8 of them."""
    R = TIER_RADIUS[tier]
    return math.log2(2 * R + 1) + 16.0 / GROUP


def quant_dequant(x: torch.Tensor, tier: str = "rk4v4") -> torch.Tensor:
    """Value map of the tier: scale = fp16(amax / R) per 64 values, snap to E8 in blocks of eight, clamp, rescale."""
    R = TIER_RADIUS[tier]
    shape = x.shape
    if shape[-1] % GROUP:
        raise ValueError("last dimension must be a multiple of 64")
    g = x.to(torch.float32).reshape(-1, shape[-1] // GROUP, GROUP)
    scale = (g.abs().amax(-1, keepdim=True) / R).to(torch.float16).to(torch.float32)
    inv = torch.where(scale > 0, 1.0 / torch.where(scale > 0, scale, torch.ones_like(scale)), torch.zeros_like(scale))
    u = (g * inv).reshape(-1, shape[-1] // 8, 8)
    p = nearest_e8(u)
    # a point pushed outside the cube by the parity fix is pulled back one lattice step along that coordinate
    over = p.abs() > R
    if bool(over.any()):
        p = torch.where(over, p - 2.0 * torch.sign(p), p)      # +-2 along one axis keeps both the coset and the parity
    return (p.reshape(-1, shape[-1] // GROUP, GROUP) * scale).reshape(shape)


def scalar_quant_dequant(x: torch.Tensor, levels: int) -> torch.Tensor:
    """Cubic-lattice baseline at the same scale rule: round to `levels` uniform steps per value (symmetric)."""
    shape = x.shape
    R = (levels - 1) / 2.0
    g = x.to(torch.float32).reshape(-1, shape[-1] // GROUP, GROUP)
    scale = (g.abs().amax(-1, keepdim=True) / R).to(torch.float16).to(torch.float32)
    inv = torch.where(scale > 0, 1.0 / torch.where(scale > 0, scale, torch.ones_like(scale)), torch.zeros_like(scale))
    return (torch.clamp(torch.round(g * inv), -R, R) * scale).reshape(shape)
