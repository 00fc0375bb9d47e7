"""Host KV arena: extent allocation, coalescing, stale handles; native and Python bookkeeping agree."""
import gc
import random

import pytest
import torch

from ninfer_fusion_b200.runtime.host_arena import GRANULE, HostKvArena


@pytest.mark.parametrize("native", [True, False])
def test_alloc_free_coalesce(native):
    a = HostKvArena(16 * GRANULE, pin=False, use_native=native)
    if native and not a.native:
        pytest.skip("native library not built")
    h1, t1 = a.alloc(3 * GRANULE)
    h2, t2 = a.alloc(GRANULE + 1)           # rounds up to two granules
    h3, t3 = a.alloc(4 * GRANULE)
    assert (h1[0], h2[0], h3[0]) == (0, 3 * GRANULE, 5 * GRANULE)
    assert t2.numel() == GRANULE + 1 and a.used == 9 * GRANULE and a.live_extents == 3
    t1.fill_(7)
    assert int(a.buffer[0]) == 7 and int(a.buffer[3 * GRANULE - 1]) == 7
    assert a.alloc(8 * GRANULE) is None     # largest free run is 7 granules
    assert a.largest_free == 7 * GRANULE
    a.free(h2)
    a.free(h1)                              # merges with the run freed before it
    assert a.largest_free == 7 * GRANULE and a.used == 4 * GRANULE
    h4, _ = a.alloc(5 * GRANULE)
    assert h4[0] == 0
    with pytest.raises(RuntimeError):
        a.free(h1)                          # stale generation
    a.free(h3)
    a.free(h4)
    assert a.used == 0 and a.largest_free == 16 * GRANULE and a.peak == 9 * GRANULE


def test_native_and_python_bookkeeping_agree():
    nat, py = HostKvArena(256 * GRANULE, pin=False, use_native=True), HostKvArena(256 * GRANULE, pin=False, use_native=False)
    if not nat.native:
        pytest.skip("native library not built")
    rng = random.Random(0)
    live = []
    for _ in range(400):
        if live and rng.random() < 0.45:
            hn, hp = live.pop(rng.randrange(len(live)))
            nat.free(hn)
            py.free(hp)
        else:
            n = rng.randrange(1, 20 * GRANULE)
            rn, rp = nat.alloc(n), py.alloc(n)
            assert (rn is None) == (rp is None)
            if rn is not None:
                assert rn[0][0] == rp[0][0]
                live.append((rn[0], rp[0]))
        assert nat.used == py.used and nat.largest_free == py.largest_free


def test_alloc_like_releases_on_garbage_collection():
    a = HostKvArena(64 * GRANULE, pin=False)
    t = a.alloc_like(torch.zeros((3, 100), dtype=torch.bfloat16))
    assert t.shape == (3, 100) and t.dtype == torch.bfloat16 and a.live_extents == 1
    del t
    gc.collect()
    assert a.live_extents == 0 and a.used == 0
    assert a.alloc_like(torch.zeros(1 << 20)) is None
