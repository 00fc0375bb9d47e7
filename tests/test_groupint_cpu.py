"""GroupIntWeight on the CPU: the encoded object round-trips through the artifact decoder and the oracle linear."""
import pytest
import torch

from ninfer_fusion_b200.artifact import layouts as L
from ninfer_fusion_b200.ops import groupint as G


@pytest.mark.parametrize("fmt", ["q4", "q5", "q6", "w8"])
def test_weight_object_roundtrip(fmt):
    g = torch.Generator().manual_seed(5)
    w = torch.randn((48, 200), generator=g) * 0.1          # K = 200: planes are padded to 256 columns
    gw = G.GroupIntWeight.from_dense(w, fmt, device="cpu")
    long_name = G.SHORT_NAMES[fmt]
    assert gw.nbytes() == L.encoded_size(long_name, "row-split-k128-v1", (48, 200))
    rep = gw.dequant()
    qmax = L.GROUP_FORMATS[long_name][4]
    group = L.GROUP_FORMATS[long_name][1]
    # every value is within half a step of its group's scale
    pad = torch.zeros((48, 256)); pad[:, :200] = w
    step = (pad.reshape(48, -1, group).abs().amax(-1) / qmax).repeat_interleave(group, dim=1)[:, :200]
    assert ((rep - w).abs() <= 0.5 * step * 1.002 + 1e-7).all()
    assert not gw.usable_by_kernel()                         # K = 200 is not a multiple of 64: the model decodes it
    x = torch.randn((3, 200), generator=g).to(torch.bfloat16)
    y = G.linear_reference(x, gw)
    assert torch.allclose(y, x.float() @ rep.t())


def test_payload_size_is_checked():
    with pytest.raises(ValueError, match="cannot hold"):
        G.GroupIntWeight("Q4G64_F16S", torch.zeros(100, dtype=torch.uint8), (64, 128))
    with pytest.raises(ValueError, match="not a groupwise-int format"):
        G.GroupIntWeight("NVFP4", torch.zeros(100, dtype=torch.uint8), (64, 128))
