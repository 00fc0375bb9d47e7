"""Device cold-slot kernels against the host codec (kv/cold_codec.py): same slot bytes, same restored planes."""
import pytest
import torch

from ninfer_fusion_b200.kv import cold_codec as C

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ninfer_fusion_b200._lib import load_native
    return load_native()


def _planes(n_slots, rows, dim, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.clamp(torch.round(torch.randn((n_slots * rows, dim), generator=g) * 45), -127, 127).to(torch.int8)
    scales = (torch.rand((n_slots * rows, dim // 64), generator=g) * 0.02 + 1e-3).to(torch.float16)
    return codes, scales


@pytest.mark.parametrize("n_slots,rows,dim", [(1, 64, 256), (5, 64, 256), (3, 16, 128)])
def test_pack_matches_the_host_codec(ops, n_slots, rows, dim):
    codes, scales = _planes(n_slots, rows, dim, n_slots + rows)
    slots = ops.cold_slot_pack_int8(codes.cuda(), scales.cuda(), rows)
    torch.cuda.synchronize()
    assert tuple(slots.shape) == (n_slots, C.cold_slot_bytes(rows, dim))
    dev = slots.cpu().numpy()
    same = total = 0
    for s in range(n_slots):
        host = C.requant_int8_g64(codes[s * rows:(s + 1) * rows], scales[s * rows:(s + 1) * rows])
        d = dev[s].tobytes()
        assert d[:16] == host[:16]                                            # header: magic, rows, dim
        same += sum(a == b for a, b in zip(d, host)); total += len(host)
        # what the device slot decodes to is what the host slot decodes to (up to rare rounding-boundary codes)
        rd, rh = C.restore_cold_slot(d), C.restore_cold_slot(host)
        assert (rd - rh).abs().max() <= 0.26 * rh.abs().max() and ((rd - rh) != 0).float().mean() < 2e-3
    assert same / total > 0.998


def test_restore_kernels_match_the_host_codec(ops):
    n_slots, rows, dim = 4, 64, 256
    codes, scales = _planes(n_slots, rows, dim, 9)
    slots = ops.cold_slot_pack_int8(codes.cuda(), scales.cuda(), rows)
    c2, s2 = ops.cold_slot_restore_int8(slots, rows, dim)
    bf = ops.cold_slot_restore_bf16(slots, rows, dim)
    torch.cuda.synchronize()
    assert c2.dtype == torch.int8 and s2.dtype == torch.float16 and bf.dtype == torch.bfloat16
    for s in range(n_slots):
        blob = slots[s].cpu().numpy().tobytes()
        want = C.restore_cold_slot(blob)
        got_bf = bf[s * rows:(s + 1) * rows].float().cpu()
        assert torch.equal(got_bf, want.to(torch.bfloat16).float())           # e2m1 x e4m3 products are exact in bf16? checked
        hc, hs = C.restore_int8_g64(blob)
        assert torch.equal(s2[s * rows:(s + 1) * rows].cpu(), hs)
        assert (c2[s * rows:(s + 1) * rows].cpu().int() - hc.int()).abs().max() <= 1
    # the round trip is lossy by construction, inside the nvfp4 envelope
    a = codes.float().reshape(-1, dim // 64, 64) * scales.float()[..., None]
    b = c2.cpu().float().reshape(-1, dim // 64, 64) * s2.cpu().float()[..., None]
    assert ((a - b) ** 2).sum() / (a ** 2).sum() < 0.02
    with pytest.raises(RuntimeError, match="slot_bytes"):
        ops.cold_slot_restore_bf16(slots[:, :-1].contiguous(), rows, dim)


def test_pages_leave_and_reenter_the_pool_as_slots(ops):
    """PagedKvCache with cold_slots: int8 layers export requantised slots (about 0.55 of the raw bytes), the other
    layers export their planes unchanged; imported pages are close to the originals (int8) or identical (bf16)."""
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.runtime.kv_cache import PagedKvCache
    from dataclasses import replace
    cfg = replace(TINY_DENSE, name="tiny-2attn", n_layers=8)              # two attention layers
    kv = PagedKvCache(cfg, 12, 64, 2, 6, "cuda", formats=["int8", "bf16"])
    g = torch.Generator().manual_seed(4)
    l0, l1 = kv.layers
    l0.k_codes.copy_(torch.clamp(torch.round(torch.randn(l0.k_codes.shape, generator=g) * 40), -127, 127).to(torch.int8).view(torch.uint8))
    l0.v_codes.copy_(torch.clamp(torch.round(torch.randn(l0.v_codes.shape, generator=g) * 40), -127, 127).to(torch.int8).view(torch.uint8))
    for sc in (l0.k_scales, l0.v_scales):
        n = sc.numel() // 2
        sc.copy_((torch.rand(n, generator=g) * 0.02 + 1e-3).to(torch.float16).view(torch.uint8).reshape(sc.shape))
    l1.k_codes.copy_(torch.randint(0, 255, l1.k_codes.shape, generator=g, dtype=torch.uint8))
    l1.v_codes.copy_(torch.randint(0, 255, l1.v_codes.shape, generator=g, dtype=torch.uint8))
    pages = [kv.pool.alloc() for _ in range(3)]
    plain = kv.export_pages(pages)
    kv.cold_slots = True
    lossy = kv.export_pages(pages)
    raw_int8 = sum(t.numel() for t in plain[:4])
    assert len(plain) == 6 and len(lossy) == 4                           # [k, v, ks, vs] + [k, v]  vs  [k slots, v slots] + [k, v]
    assert sum(t.numel() for t in lossy[:2]) < 0.56 * raw_int8
    assert torch.equal(lossy[2], plain[4]) and torch.equal(lossy[3], plain[5])
    back = kv.import_pages(lossy, 3)
    assert back is not None and len(back) == 3
    src, dst = torch.tensor(pages, device="cuda"), torch.tensor(back, device="cuda")
    assert torch.equal(l1.k_codes[dst], l1.k_codes[src]) and torch.equal(l1.v_codes[dst], l1.v_codes[src])

    def values(codes, scales, idx):
        c = codes[idx].view(torch.int8).float()
        s = scales[idx].view(torch.float16).float()
        return c.reshape(*c.shape[:-1], -1, 64) * s[..., None]
    for codes, scales in ((l0.k_codes, l0.k_scales), (l0.v_codes, l0.v_scales)):
        a, b = values(codes, scales, src), values(codes, scales, dst)
        assert float(((a - b) ** 2).sum() / (a ** 2).sum()) < 0.02
