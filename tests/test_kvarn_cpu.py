"""KVarN k4v2 tile codec oracle: record arithmetic, error envelope, what stays bf16."""
import torch

from ninfer_fusion_b200.kv import kvarn as KV


def test_record_size_matches_the_profile():
    assert KV.record_bytes(256, 128) == 26880 and KV.record_bytes(256, 128) % 256 == 0
    assert abs(KV.bits_per_value(256, 128) - 3.28125) < 1e-9


def test_tile_codec_error_and_balancing():
    g = torch.Generator().manual_seed(0)
    k = torch.randn((128, 256), generator=g)
    k[:, [3, 70]] *= 9.0                                   # loud channels
    k[5] *= 6.0                                            # a loud token
    v = torch.randn((128, 256), generator=g)
    kq, vq = KV.quant_dequant_tile(k, v)
    ek = float(((kq - k) ** 2).sum() / (k ** 2).sum())
    ev = float(((vq - v) ** 2).sum() / (v ** 2).sum())
    assert ek < 0.02 and ev < 0.35                          # 4-bit K; 2-bit min-max V: step^2 / 12 of a +-2.8 sigma range
    # without the two-sided balancing the loud rows and columns eat the 4-bit range of everything else
    plain = KV._asym(k, 16, dim=0)
    quiet = torch.ones(256, dtype=torch.bool); quiet[[3, 70]] = False
    rows = torch.ones(128, dtype=torch.bool); rows[5] = False
    e_bal = float(((kq - k)[rows][:, quiet] ** 2).mean())
    e_plain = float(((plain - k)[rows][:, quiet] ** 2).mean())
    assert e_bal < e_plain


def test_sink_and_tail_stay_exact():
    g = torch.Generator().manual_seed(1)
    n = 16 + 2 * 128 + 37
    k, v = torch.randn((n, 2, 128), generator=g), torch.randn((n, 2, 128), generator=g)
    kq, vq = KV.quant_dequant_sequence(k, v, sink=16)
    assert torch.equal(kq[:16], k[:16]) and torch.equal(vq[:16], v[:16])
    assert torch.equal(kq[16 + 256:], k[16 + 256:]) and torch.equal(vq[16 + 256:], v[16 + 256:])
    mid = slice(16, 16 + 256)
    assert not torch.equal(kq[mid], k[mid]) and float((kq[mid] - k[mid]).abs().max()) < 0.6
    short_k, short_v = KV.quant_dequant_sequence(k[:100], v[:100])
    assert torch.equal(short_k, k[:100]) and torch.equal(short_v, v[:100])          # no complete tile yet
