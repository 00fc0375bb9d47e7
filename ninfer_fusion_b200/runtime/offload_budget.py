"""When moving weights off the device pays, as arithmetic.

Per decode round every resident weight is read once (constant in the context) and the whole KV of every sequence is
read once (linear in the context).  Weights that live in pinned host memory are re-fetched over the host link every
round, so off-loading never makes a round faster: it is worthwhile only when the alternative is that the request does
not fit at all, and its price is `offloaded_bytes / link_bandwidth` per round (hidden behind the round only as far as
the link is faster than the round needs).  These are pure functions over plain numbers: the residency planner
(`runtime/weight_offload.py`) decides WHICH layers move, this decides WHETHER and what it costs.

* `KvCapacityFit`: KV device bytes = bytes_per_token_bit x tokens x bits + constant, solved exactly from two observed
  points (no fitted-looking constant is typed here); `bits_within` answers "which average KV precision fits in what is
  left".
* `offload_verdict`: resident / offload / does-not-fit for a model, a context and a device, with the bytes that have to
  move and the milliseconds per round they cost.

Reference: src/product/weight_offload_budget.h (transfer math as a pure function, the affine KV capacity model),
src/product/weight_residency.h.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class KvCapacityPoint:
    tokens: int
    nbytes: int
    bits_per_element: float


@dataclass(frozen=True)
class KvCapacityFit:
    bytes_per_token_bit: float
    constant_bytes: float

    @staticmethod
    def from_points(a: KvCapacityPoint, b: KvCapacityPoint) -> "KvCapacityFit":
        xa, xb = a.tokens * a.bits_per_element, b.tokens * b.bits_per_element
        if xa == xb:
            raise ValueError("the two capacity points must differ in tokens x bits")
        slope = (b.nbytes - a.nbytes) / (xb - xa)
        return KvCapacityFit(slope, a.nbytes - slope * xa)

    def bytes_for(self, tokens: int, bits: float) -> float:
        return self.bytes_per_token_bit * tokens * bits + self.constant_bytes

    def bits_within(self, tokens: int, available_bytes: float) -> float:
        span = self.bytes_per_token_bit * tokens
        return 0.0 if span <= 0 else (available_bytes - self.constant_bytes) / span


@dataclass(frozen=True)
class OffloadVerdict:
    state: str                    # "resident" | "offload" | "does_not_fit"
    offloaded_bytes: int = 0
    added_ms_per_round: float = 0.0
    kv_bytes: int = 0
    note: str = ""


def offload_verdict(weight_bytes: int, kv_bytes: int, other_bytes: int, device_bytes: int, host_link_gbs: float = 50.0,
                    host_bytes: Optional[int] = None, min_resident_fraction: float = 0.1) -> OffloadVerdict:
    """Everything resident when it fits; else the smallest amount of weights that has to live on the host, its price
    per decode round on a `host_link_gbs` GB/s link, or "does not fit" when even `min_resident_fraction` of the
    weights plus the KV exceed the device (or the host cannot hold what must move)."""
    need = weight_bytes + kv_bytes + other_bytes
    if need <= device_bytes:
        return OffloadVerdict("resident", 0, 0.0, kv_bytes, "weights and KV fit: resident weights are strictly faster")
    move = need - device_bytes
    if move > weight_bytes * (1.0 - min_resident_fraction):
        return OffloadVerdict("does_not_fit", 0, 0.0, kv_bytes,
                              "the KV alone leaves no room for a working share of the weights: lower the KV precision, "
                              "shorten the context or shard the model")
    if host_bytes is not None and move > host_bytes:
        return OffloadVerdict("does_not_fit", 0, 0.0, kv_bytes, "the host cannot hold the weights that would have to move")
    ms = move / (host_link_gbs * 1e9) * 1e3
    return OffloadVerdict("offload", int(move), ms, kv_bytes,
                          f"{move / (1 << 30):.1f} GiB of weights re-fetched every round over the host link")
