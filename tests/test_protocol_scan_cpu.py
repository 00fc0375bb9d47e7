"""Every interleaving of the push / counter protocol: safe with the kernels' two parity buffers, unsafe with one."""
import pytest

from ninfer_fusion_b200.parallel.protocol_scan import scan


@pytest.mark.parametrize("world,calls", [(2, 4), (3, 3)])
def test_parity_buffers_are_safe_in_every_interleaving(world, calls):
    violation, states = scan(world=world, calls=calls, depth=2)
    assert violation is None and states > 100


def test_a_single_buffer_is_overwritten_early():
    violation, _ = scan(world=2, calls=2, depth=1)
    assert violation is not None and violation.kind == "stale_read" and violation.call == 0
    assert "calls" in violation.detail


def test_missing_arrival_is_reported_as_deadlock():
    # a world of 2 whose consumer expects 3 arrivals per call can never proceed
    import ninfer_fusion_b200.parallel.protocol_scan as P
    orig = P._program

    def short(rank, world, calls):
        steps = orig(rank, world, calls)
        return [s for s in steps if not (s[0] == "add" and s[1] != rank and rank == 1)]   # rank 1 never signals rank 0
    P._program = short
    try:
        violation, _ = scan(world=2, calls=1, depth=2)
    finally:
        P._program = orig
    assert violation is not None and violation.kind == "deadlock" and violation.rank == 0


def test_expert_parallel_protocol_needs_the_unconditional_arrival():
    """Single-buffered counts and receive rows are safe because every push signals every rank, rows or not; if a rank
    only signalled the ranks it sent rows to, a rank with no traffic to a slow peer could lap it and overwrite its
    counts."""
    from ninfer_fusion_b200.parallel.protocol_scan import expert_parallel_programs, scan_programs
    local_only = [[True, False], [False, True]]                       # every token stays on its own rank
    dense = [[True, True], [True, True]]
    mixed = [[True, True, False], [False, True, True], [True, False, True]]
    for rows, world in ((local_only, 2), (dense, 2), (mixed, 3)):
        v, states = scan_programs(expert_parallel_programs(world, 3 if world == 2 else 2, rows, unconditional_arrive=True))
        assert v is None and states > 50, (rows, v)
    v, _ = scan_programs(expert_parallel_programs(2, 2, local_only, unconditional_arrive=False))
    assert v is not None and v.kind == "stale_read"
    v, _ = scan_programs(expert_parallel_programs(2, 3, dense, unconditional_arrive=False))
    assert v is None                                                   # with traffic between every pair the waits chain anyway
