"""E8-lattice quantiser: membership, exact nearest point, gain over the cubic lattice, tier widths."""
import itertools

import pytest
import torch

from ninfer_fusion_b200.kv import e8_lattice as E8


def test_points_are_lattice_points_and_nearest():
    g = torch.Generator().manual_seed(0)
    x = torch.randn((400, 8), generator=g) * 2.5
    p = E8.nearest_e8(x)
    assert bool(E8.in_e8(p).all())
    # no lattice point near p is closer: the 240 minimal vectors of E8 are the neighbours to try
    mins = []
    for i, j in itertools.combinations(range(8), 2):
        for si in (1.0, -1.0):
            for sj in (1.0, -1.0):
                v = torch.zeros(8); v[i], v[j] = si, sj
                mins.append(v)
    for signs in itertools.product((0.5, -0.5), repeat=8):
        if sum(s < 0 for s in signs) % 2 == 0:
            mins.append(torch.tensor(signs))
    M = torch.stack(mins)
    assert M.shape == (240, 8) and bool(E8.in_e8(M).all())
    d0 = (x - p).pow(2).sum(-1)
    dn = (x[:, None, :] - (p[:, None, :] + M[None])).pow(2).sum(-1).min(-1).values
    assert bool((d0 <= dn + 1e-5).all())
    assert not bool(E8.in_e8(torch.tensor([[1.0, 0, 0, 0, 0, 0, 0, 0]])).any())      # odd sum
    assert not bool(E8.in_e8(torch.tensor([[0.5, 0, 0, 0, 0, 0, 0, 0.5]])).any())    # mixed cosets
    with pytest.raises(ValueError):
        E8.nearest_e8(torch.zeros(3, 4))


def test_gain_over_the_cubic_lattice_at_equal_density():
    """Both lattices have one point per unit volume; on a smooth source E8's error is about 0.65 dB lower."""
    g = torch.Generator().manual_seed(1)
    x = torch.rand((20000, 8), generator=g) * 40 - 20
    e8 = (x - E8.nearest_e8(x)).pow(2).mean()
    z8 = (x - torch.round(x)).pow(2).mean()
    gain_db = 10 * torch.log10(z8 / e8)
    assert 0.5 < float(gain_db) < 0.8


def test_tier_value_map_and_widths():
    g = torch.Generator().manual_seed(2)
    k = torch.randn((64, 2, 256), generator=g)
    err = {}
    for tier in ("rk4v4", "rk3v4", "rk2v4"):
        q = E8.quant_dequant(k, tier)
        assert q.shape == k.shape
        R = E8.TIER_RADIUS[tier]
        scale = (k.reshape(-1, 4, 64).abs().amax(-1) / R).to(torch.float16).float()
        units = q.reshape(-1, 4, 64) / scale[..., None]
        assert float(units.abs().max()) <= R + 1e-3
        assert bool(E8.in_e8(units.reshape(-1, 8)).all())
        err[tier] = float((q - k).pow(2).mean() / k.pow(2).mean())
    assert err["rk4v4"] < err["rk3v4"] < err["rk2v4"] and err["rk4v4"] < 0.01
    assert abs(E8.bits_per_value("rk4v4") - 4.25) < 1e-9 and abs(E8.bits_per_value("rk3v4") - 3.25) < 1e-9
    # same scale rule, same 16 levels per value: the lattice beats scalar rounding on Gaussian rows
    scalar = float((E8.scalar_quant_dequant(k, 16) - k).pow(2).mean() / k.pow(2).mean())
    assert err["rk4v4"] < scalar
    with pytest.raises(ValueError):
        E8.quant_dequant(torch.zeros(4, 100))
