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
device; the reference keeps the same kind of scan for its 2-rank
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


# ------------------------------------------------------------------------------------------------ generic engine
def scan_programs(progs: List[List[Tuple]], max_states: int = 2_000_000) -> Tuple[Optional[Violation], int]:
    """Every interleaving of per-rank step lists over shared cells.  Steps:
    ("store", cell, value) | ("add", counter) | ("wait", counter, threshold) | ("read", [cells], expected, rank, call)."""
    cells = sorted({s[1] for p in progs for s in p if s[0] == "store"} | {c for p in progs for s in p if s[0] == "read" for c in s[1]})
    counters = sorted({s[1] for p in progs for s in p if s[0] in ("add", "wait")})
    ci = {c: i for i, c in enumerate(cells)}
    ki = {c: i for i, c in enumerate(counters)}
    start = (tuple(0 for _ in progs), tuple(-1 for _ in cells), tuple(0 for _ in counters))
    seen, stack = {start}, [start]
    while stack:
        pcs, mem, cnt = stack.pop()
        if len(seen) > max_states:
            raise RuntimeError("state space larger than max_states")
        moved, finished = False, True
        for r, prog in enumerate(progs):
            if pcs[r] >= len(prog):
                continue
            finished = False
            s = prog[pcs[r]]
            n_mem, n_cnt = mem, cnt
            if s[0] == "store":
                m = list(mem); m[ci[s[1]]] = s[2]; n_mem = tuple(m)
            elif s[0] == "add":
                k = list(cnt); k[ki[s[1]]] += 1; n_cnt = tuple(k)
            elif s[0] == "wait":
                if cnt[ki[s[1]]] < s[2]:
                    continue
            else:
                got = [mem[ci[c]] for c in s[1]]
                if any(v != s[2] for v in got):
                    return Violation("stale_read", s[3], s[4], f"rank {s[3]} call {s[4]} read {got}, expected {s[2]}"), len(seen)
            moved = True
            n_pcs = list(pcs); n_pcs[r] += 1
            nxt = (tuple(n_pcs), n_mem, n_cnt)
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not moved and not finished:
            blocked = [r for r in range(len(progs)) if pcs[r] < len(progs[r])]
            return Violation("deadlock", blocked[0], -1, f"ranks {blocked} wait for counters that never advance"), len(seen)
    return None, len(seen)


def expert_parallel_programs(world: int, calls: int, rows: List[List[bool]], unconditional_arrive: bool = True) -> List[List[Tuple]]:
    """The expert-parallel layer protocol (csrc/moe/moe_route.cu): a histogram exchange that doubles as a barrier, then
    rows pushed into SINGLE receive buffers.  rows[s][d]: does rank s route any token to rank d in a call.

        plan:  store counts[d][r] for every d; add count_flag[d]; wait count_flag[r] >= (e + 1) W; read counts[r][*]
        push:  store recv[d][r] where rows[r][d]; add arrive_flag[d] (for EVERY d when `unconditional_arrive`, as the
               kernel does; only where rows were sent otherwise); wait arrive_flag[r]; read recv[r][s] for senders s

    The receive and count buffers have no parity: what keeps call e + 1 from overwriting call e is that a rank cannot
    leave call e before every rank's push kernel of call e ran, which follows that rank's plan in stream order."""
    progs = []
    for r in range(world):
        p: List[Tuple] = []
        for e in range(calls):
            for d in range(world):
                p.append(("store", ("counts", d, r), e))
            for d in range(world):
                p.append(("add", ("count_flag", d)))
            p.append(("wait", ("count_flag", r), (e + 1) * world))
            p.append(("read", [("counts", r, s) for s in range(world)], e, r, e))
            for d in range(world):
                if rows[r][d]:
                    p.append(("store", ("recv", d, r), e))
            senders = [s for s in range(world) if rows[s][r]]
            for d in range(world):
                if unconditional_arrive or rows[r][d]:
                    p.append(("add", ("arrive_flag", d)))
            expect = world if unconditional_arrive else len(senders)
            p.append(("wait", ("arrive_flag", r), (e + 1) * expect))
            if senders:
                p.append(("read", [("recv", r, s) for s in senders], e, r, e))
        progs.append(p)
    return progs
