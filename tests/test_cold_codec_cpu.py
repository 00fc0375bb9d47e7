"""Cold-slot codecs: rANS coder (native and Python twin, byte-identical), lossy cold slot, disk-tier file format."""
import importlib
import os

import numpy as np
import pytest
import torch

from ninfer_fusion_b200.kv import cold_codec as C


def _peaked_nibbles(n, seed):
    rng = np.random.default_rng(seed)
    v = np.clip(np.rint(rng.normal(8, 1.5, 2 * n)), 0, 15).astype(np.uint8)
    return (v[0::2] | (v[1::2] << 4)).astype(np.uint8)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("n", [0, 1, 7, 1000, 9216])
def test_rans_roundtrip_and_twin_identity(bits, n):
    data = _peaked_nibbles(n, n + bits) if bits == 4 else \
        np.random.default_rng(n).normal(0, 12, n).astype(np.int8).view(np.uint8)
    blob = C.rans_encode(data, bits)
    assert C.rans_decode(blob) == data.tobytes()
    twin = C._py_encode(np.ascontiguousarray(data), bits, C.rans_bound(data.size, bits))
    assert twin == blob                      # the native coder and the Python twin write the same stream
    assert C._py_decode(blob) == data.tobytes()
    if n >= 1000:
        assert len(blob) < 0.85 * n + 10 + 2 * (1 << bits)   # peaked sources compress


def test_rans_budget_and_malformed_streams():
    noise = np.random.default_rng(1).integers(0, 256, 4096, dtype=np.uint8)
    assert C.rans_encode(noise, 8, budget=int(4096 * 0.95)) is None          # incompressible: over budget
    assert C.rans_encode(noise, 8) is not None                                # without a budget it still codes
    blob = C.rans_encode(np.zeros(500, dtype=np.uint8), 8)
    assert len(blob) < 540 and C.rans_decode(blob) == bytes(500)              # one symbol: a table and a flush
    with pytest.raises(ValueError, match="bad magic"):
        C.rans_decode(b"X" + blob[1:])
    good = C.rans_encode(_peaked_nibbles(2000, 3), 4)
    with pytest.raises(ValueError, match="truncated"):
        C.rans_decode(good[:-40])
    bad = bytearray(good); bad[10] ^= 0x40                                    # frequency table no longer sums to 4096
    with pytest.raises(ValueError, match="frequency table"):
        C.rans_decode(bytes(bad))
    with pytest.raises(ValueError):
        C.rans_encode(noise, 5)


def test_cold_slot_layout_error_and_entropy_stage():
    torch.manual_seed(0)
    v = torch.randn(64, 256)
    v[:, 7] *= 8                                                              # an outlier channel
    slot = C.pack_cold_slot(v)
    assert len(slot) == C.cold_slot_bytes(64, 256) == 9232
    r = C.restore_cold_slot(slot)
    nmse = ((r - v) ** 2).sum().item() / (v ** 2).sum().item()
    assert nmse < 0.02
    stream, _ = C.code_cold_slot(slot)
    assert len(stream) <= len(slot) + 10 and C.decode_cold_slot(stream) == slot
    # a smooth page (most values small against their group's maximum) does compress
    smooth = torch.randn(64, 256) * 0.05
    smooth[:, ::16] = 3.0
    s2 = C.pack_cold_slot(smooth)
    st2, coded = C.code_cold_slot(s2)
    assert coded and len(st2) < 0.8 * len(s2) and C.decode_cold_slot(st2) == s2
    with pytest.raises(ValueError):
        C.restore_cold_slot(slot[:-1])


def test_int8_tier_through_the_cold_slot():
    g = torch.Generator().manual_seed(2)
    codes = torch.clamp(torch.round(torch.randn((64, 256), generator=g) * 40), -127, 127).to(torch.int8)
    scales = (torch.rand((64, 4), generator=g) * 0.02 + 0.001).to(torch.float16)
    slot = C.requant_int8_g64(codes, scales)
    c2, s2 = C.restore_int8_g64(slot)
    assert c2.dtype == torch.int8 and s2.dtype == torch.float16 and c2.abs().max() <= 127
    a = codes.float().reshape(64, 4, 64) * scales.float()[..., None]
    b = c2.float().reshape(64, 4, 64) * s2.float()[..., None]
    assert ((a - b) ** 2).sum().item() / (a ** 2).sum().item() < 0.02         # the slot is lossy by construction


def test_python_twin_is_used_without_the_library(monkeypatch):
    monkeypatch.setenv("NFB200_PY_RANS", "1")
    mod = importlib.reload(C)
    try:
        assert not mod.native_available()
        data = _peaked_nibbles(300, 9)
        assert mod.rans_decode(mod.rans_encode(data, 4)) == data.tobytes()
    finally:
        monkeypatch.delenv("NFB200_PY_RANS")
        importlib.reload(C)


def test_disk_tier_writes_coded_frontiers(tmp_path):
    """ProgramBase's disk tier with cold_entropy: the file is smaller than the raw tensors and revives bit-exactly."""
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.runtime.program import Checkpoint, ProgramBase

    class Stub(ProgramBase):
        def __init__(self):
            super().__init__(TINY_DENSE, max_lanes=2, max_context=64)
            self.revived = None

        def _demote(self, handle):
            return {"n_pages": 2, "tensors": [handle, [torch.arange(12.0).reshape(3, 4)]]}

        def _promote(self, cold):
            self.revived = cold
            return ("hot", cold["n_pages"])

        def _drop(self, handle):
            pass

    p = Stub()
    p.host_budget_bytes, p.disk_budget_bytes, p.cold_dir, p.cold_entropy = 1, 1 << 30, str(tmp_path / "cold"), True
    g = torch.Generator().manual_seed(4)
    planes = [torch.clamp(torch.round(torch.randn((2, 64, 2, 256), generator=g) * 10), -127, 127).to(torch.int8),
              torch.rand((2, 64, 2, 4), generator=g).to(torch.float16)]
    fields = {f.name for f in Checkpoint.__dataclass_fields__.values()}
    kw = dict(session="s", tokens=[1, 2, 3], kind="turn", handle=planes, last_used=1)
    ck = Checkpoint(**{k: v for k, v in kw.items() if k in fields})
    p.checkpoints.append(ck)
    assert p._evict_checkpoint()
    assert ck.tier == "disk" and p.cold_stats["demoted_disk"] == 1
    assert p.cold_stats["disk_stored_bytes"] < 0.9 * p.cold_stats["disk_raw_bytes"]
    assert os.path.getsize(ck.handle["path"]) < 0.92 * p.cold_stats["disk_raw_bytes"]
    assert p._warm_up(ck) and ck.tier == "gpu"
    got = p.revived["tensors"]
    assert torch.equal(got[0][0], planes[0]) and torch.equal(got[0][1], planes[1]) and got[0][1].dtype == torch.float16
    assert torch.equal(got[1][0], torch.arange(12.0).reshape(3, 4))


def test_a_failed_spill_is_counted_not_fatal(tmp_path):
    """The disk tier's directory cannot be created (a file sits where it should be): the frontier is dropped and
    counted, nothing raises."""
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.runtime.program import Checkpoint, ProgramBase

    class Stub(ProgramBase):
        def _demote(self, handle):
            return {"n_pages": 1, "tensors": [[torch.zeros(64)]]}

        def _drop(self, handle):
            pass

    blocker = tmp_path / "not-a-dir"
    blocker.write_text("x")
    p = Stub(TINY_DENSE, max_lanes=2, max_context=64)
    p.host_budget_bytes, p.disk_budget_bytes, p.cold_dir = 1, 1 << 30, str(blocker / "cold")
    ck = Checkpoint("s", "turn", [1, 2, 3], object(), last_used=1)
    p.checkpoints.append(ck)
    assert p._evict_checkpoint()
    assert ck not in p.checkpoints
    assert p.cold_stats["spill_write_failed"] == 1 and p.cold_stats["dropped"] == 1 and p.cold_stats["demoted_disk"] == 0
