"""Block Hadamard rotation of a matmul's input dimension, folded into the weights.

For the normalised Hadamard matrix H of a block (H H^T = I) and a weight W [N, K] whose K axis is cut into blocks,
``x W^T = (x H)(W H)^T``.  ``fold`` rotates the weight once, before it is quantised; the activation side is rotated
at run time by ``torch.ops.nfb200.hadamard_blocks`` (csrc/pointwise/hadamard.cu).  Rotating spreads an outlier input
channel over its block, so a group scale is no longer dictated by one loud column and 4-bit codes keep more of the
other 63.  Reference: prism_fold (rotation folded into the weights) and e8act (activation-side 64-point Hadamard)
under src/ops/linear.
"""
from __future__ import annotations

import torch

from . import reference as R

BLOCKS = (64, 128, 256)


def _check(K: int, block: int) -> None:
    if block not in BLOCKS:
        raise ValueError(f"rotation block must be one of {BLOCKS}")
    if K % block:
        raise ValueError(f"input width {K} is not a multiple of the rotation block {block}")


def fold(w: torch.Tensor, block: int = 64) -> torch.Tensor:
    """W -> W H (block diagonal over the input dimension), fp32 arithmetic, dtype and device of `w`."""
    N, K = w.shape
    _check(K, block)
    H = R.hadamard_matrix(block).to(w.device, torch.float32)
    return (w.to(torch.float32).reshape(N, K // block, block) @ H).reshape(N, K).to(w.dtype)


def rotate_reference(x: torch.Tensor, block: int = 64) -> torch.Tensor:
    """Oracle of the activation-side rotation: x H per block, fp32."""
    T, K = x.shape
    _check(K, block)
    H = R.hadamard_matrix(block).to(x.device, torch.float32)
    return (x.to(torch.float32).reshape(T, K // block, block) @ H).reshape(T, K)


def rotate(ops, x: torch.Tensor, block: int = 64, out: torch.Tensor = None) -> torch.Tensor:
    """Device rotation of bf16 rows (in place when out is x)."""
    _check(x.shape[1], block)
    if out is None:
        out = torch.empty_like(x)
    ops.hadamard_blocks(x, out, block)
    return out
