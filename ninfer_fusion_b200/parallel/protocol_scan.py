"""Exhaustive interleaving scan of the push / counter protocol the fused tensor-parallel kernels use.

Model of one reduce call `e` on rank `r` (csrc/gemm: push-all epilogue; csrc/comm/tp_kernels.cu: tp_sum_norm):

    for every destination d:   store  recv[d][e % depth][r] = payload(r, e)      (plain peer store)
    for every destination d:   add 1  flag[d]                                    (red.release: ordered after r's stores)
    wait  flag[r] >= (e + 1) * W                                                 (ld.acquire, bounded on the device)
    read  recv[r][e % depth][*]                                                  and sum

Counters only grow, waits are `>=`, and a buffer is reused by call e + depth.  The scan walks EVERY interleaving of
those steps between the ranks (stores and adds to different destinations are separate steps) and checks that a
consumer always reads the payloads of its own call (nothing stale, nothing overwritten early) and that no schedule
deadlocks.  With depth = 2 (the kernels' parity buffers) the protocol is safe; with depth = 1 the scan finds the
overwrite, which is why the parity exists.  This is the host-side proof that stands in for a race detector on the
device (compute-sanitizer is not available on the pool); the reference keeps the same kind of scan for its 2-rank
transport (src/core/tp_transport.h: ordering scan of the slot protocol).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class Violation:
    kind: str                 # "stale_read" | "deadlock"
    rank: int
    call: int
    detail: str


def _program(rank: int, world: int, calls: int) -> List[Tuple]:
    steps: List[Tuple] = []
    for e in range(calls):
        for d in range(world):
            steps.append(("store", d, e))
        for d in range(world):
            steps.append(("add", d, e))
        steps.append(("consume", rank, e))
    return steps


def scan(world: int = 2, calls: int = 3, depth: int = 2, max_states: int = 2_000_000) -> Tuple[Optional[Violation], int]:
    """Returns (first violation or None, number of distinct states visited)."""
    progs = [_program(r, world, calls) for r in range(world)]
    # recv[d][slot][src] = call whose payload sits there (-1 = nothing yet); flags[d] = arrivals so far
    recv0 = tuple(tuple(tuple(-1 for _ in range(world)) for _ in range(depth)) for _ in range(world))
    start = (tuple(0 for _ in range(world)), recv0, tuple(0 for _ in range(world)))
    seen = {start}
    stack = [start]
    while stack:
        pcs, recv, flags = stack.pop()
        if len(seen) > max_states:
            raise RuntimeError("state space larger than max_states")
        moved = False
        finished = True
        for r in range(world):
            if pcs[r] >= len(progs[r]):
                continue
            finished = False
            op, d, e = progs[r][pcs[r]]
            n_recv, n_flags = recv, flags
            if op == "store":
                slot = e % depth
                row = list(recv[d][slot]); row[r] = e
                plane = list(recv[d]); plane[slot] = tuple(row)
                full = list(recv); full[d] = tuple(plane)
                n_recv = tuple(full)
            elif op == "add":
                fl = list(flags); fl[d] += 1
                n_flags = tuple(fl)
            else:  # consume: blocked until every rank's arrival of this call is counted
                if flags[r] < (e + 1) * world:
                    continue
                got = recv[r][e % depth]
                if any(v != e for v in got):
                    return Violation("stale_read", r, e, f"rank {r} call {e} read payloads of calls {list(got)}"), len(seen)
            moved = True
            n_pcs = list(pcs); n_pcs[r] += 1
            nxt = (tuple(n_pcs), n_recv, n_flags)
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not moved and not finished:
            blocked = [r for r in range(world) if pcs[r] < len(progs[r])]
            r = blocked[0]
            return Violation("deadlock", r, progs[r][pcs[r]][2], f"ranks {blocked} wait for arrivals that never come"), len(seen)
    return None, len(seen)
