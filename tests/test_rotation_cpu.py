"""Hadamard rotation folded into weights: algebra and what it buys a 4-bit group quantiser."""
import pytest
import torch

from ninfer_fusion_b200.ops import groupint as G
from ninfer_fusion_b200.ops import rotation as ROT


@pytest.mark.parametrize("block", [64, 128, 256])
def test_fold_and_rotate_cancel(block):
    g = torch.Generator().manual_seed(block)
    w = torch.randn((24, 512), generator=g)
    x = torch.randn((5, 512), generator=g)
    y = x @ w.t()
    y_rot = ROT.rotate_reference(x, block) @ ROT.fold(w, block).t()
    assert torch.allclose(y, y_rot, atol=1e-3)
    assert torch.allclose(ROT.fold(ROT.fold(w, block), block), w, atol=1e-4)      # H is its own inverse
    with pytest.raises(ValueError):
        ROT.fold(torch.zeros(4, 96), 64)
    with pytest.raises(ValueError):
        ROT.fold(torch.zeros(4, 96), 32)


def test_rotation_lowers_q4_error_when_input_channels_are_loud():
    g = torch.Generator().manual_seed(1)
    w = torch.randn((128, 1024), generator=g) * 0.02
    w[:, ::64] *= 25.0                                     # one loud input channel per group of 64
    x = torch.randn((16, 1024), generator=g).to(torch.bfloat16)
    ref = x.float() @ w.t()
    plain = G.GroupIntWeight.from_dense(w, "q4", device="cpu")
    rot = G.GroupIntWeight.from_dense(w, "q4", device="cpu", rot_block=64)
    assert rot.rot_block == 64 and plain.rot_block == 0
    e_plain = (G.linear_reference(x, plain) - ref).pow(2).mean().sqrt()
    e_rot = (G.linear_reference(x, rot) - ref).pow(2).mean().sqrt()
    assert e_rot < 0.6 * e_plain
    # the represented weight of the rotated object is W again (up to its own quantisation error)
    assert (rot.dequant() - w).abs().max() < (plain.dequant() - w).abs().max()


def test_weight_format_suffix_selects_the_rotation():
    from ninfer_fusion_b200.models.weights import quantize_tensor
    t = torch.randn(64, 256)
    a = quantize_tensor("text/layers/0/mlp/down", t, "q4+h64")
    b = quantize_tensor("text/layers/0/mlp/down", t, "q4")
    c = quantize_tensor("text/layers/0/mlp/down", torch.randn(64, 160), "q4+h64")   # 160 % 64 != 0: left unrotated
    assert a.rot_block == 64 and b.rot_block == 0 and c.rot_block == 0
