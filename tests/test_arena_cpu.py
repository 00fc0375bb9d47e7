"""Bump arena: alignment, scopes that give their bytes back, peak trace, overflow refusal, stable addresses."""
import pytest
import torch

from ninfer_fusion_b200.runtime.arena import ArenaOverflow, BumpArena


def test_scopes_reuse_bytes_and_the_peak_trace_names_what_was_live():
    a = BumpArena(64 << 10, "cpu", align=256)
    keep = a.alloc((100,), torch.float32, "keep")
    assert keep.data_ptr() % 256 == 0 and keep.numel() == 100
    with a.scope():
        t1 = a.alloc((1000,), torch.bfloat16, "layer scratch")
        p1 = t1.data_ptr()
        with a.scope():
            a.alloc((4096,), torch.uint8, "inner")
        inner_gone = a.cursor
        assert a.alloc((16,), torch.int32, "after inner").data_ptr() % 256 == 0
    assert a.cursor < inner_gone
    with a.scope():
        t2 = a.alloc((1000,), torch.bfloat16, "next layer scratch")
        assert t2.data_ptr() == p1                      # the same bytes, the same address: graph replays stay valid
    assert [l for l, _, _ in a.trace] == ["keep", "layer scratch", "inner"] and a.peak >= 400 + 2000 + 4096
    keep.fill_(3.0)
    t2.fill_(1.0)
    assert float(keep.sum()) == 300.0                    # neighbours do not overlap
    assert "peak" in a.report() and "inner" in a.report()


def test_overflow_is_refused_with_the_live_list():
    a = BumpArena(1024, "cpu", align=64)
    a.alloc((128,), torch.float32, "half")
    with pytest.raises(ArenaOverflow, match="half:512"):
        a.alloc((1024,), torch.uint8, "too much")
    a.reset()
    assert a.alloc((1024,), torch.uint8, "fits now").numel() == 1024
    with pytest.raises(ValueError):
        BumpArena(16, "cpu", align=48)
