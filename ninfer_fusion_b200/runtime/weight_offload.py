"""Weight residency under a device budget: resident layers stay on the GPU, the rest live in pinned host memory and
rotate through a small device arena, prefetched one layer ahead on a copy stream.

Counterpart of the reference's weight-residency planner + rotating arena ("W13": src/product/weight_residency.h,
weight_offload_budget.h — classify spans resident / offloaded, pinned-host store, per-layer prefetch driven by
`note_layer`).  On a 180 GB part this is for models (or co-located deployments) that do not fit; the copy of layer
i + 1 overlaps the compute of layer i, so the cost of an offloaded layer is max(compute, bytes / PCIe bandwidth).

`OffloadedWeights` is a read-only mapping that the model indexes like its plain weight dict.  Only plain tensors
rotate; quantised weight objects and everything outside the layer stack stay resident.  Decode graphs bake
addresses and cannot contain the host copies, so an offloaded model runs eagerly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Tuple

import torch


@dataclass
class ResidencyPlan:
    resident_layers: List[int]
    offloaded_layers: List[int]
    layer_bytes: Dict[int, int]
    fixed_bytes: int          # tensors outside the layer stack (always resident)
    arena_bytes: int          # slots x largest offloaded layer
    device_bytes: int         # fixed + resident layers + arena
    host_bytes: int


def _layer_of(name: str, prefix: str) -> Optional[int]:
    head = f"{prefix}/layers/"
    if not name.startswith(head):
        return None
    return int(name[len(head):].split("/", 1)[0])


def _nbytes(t) -> int:
    if isinstance(t, torch.Tensor):
        return t.numel() * t.element_size()
    return sum(_nbytes(getattr(t, a)) for a in ("codes", "scale") if isinstance(getattr(t, a, None), torch.Tensor))


def _movable(t) -> bool:
    """Only plain matrices rotate; norm vectors, gating vectors and quantised weight objects stay on the device."""
    return isinstance(t, torch.Tensor) and t.dim() >= 2


def plan_residency(weights: Dict[str, object], budget_bytes: int, prefix: str = "text", slots: int = 2) -> ResidencyPlan:
    """Everything resident if it fits; otherwise layers stay resident from the front while the budget still holds the
    fixed tensors, the resident layers and a `slots`-deep arena of the largest layer."""
    layer_bytes: Dict[int, int] = {}
    fixed = 0
    for name, t in weights.items():
        l = _layer_of(name, prefix)
        if l is None or not _movable(t):
            fixed += _nbytes(t)
        else:
            layer_bytes[l] = layer_bytes.get(l, 0) + _nbytes(t)
    layers = sorted(layer_bytes)
    total = fixed + sum(layer_bytes.values())
    if total <= budget_bytes or not layers:
        return ResidencyPlan(layers, [], layer_bytes, fixed, 0, total, 0)
    arena = slots * max(layer_bytes.values())
    used = fixed
    resident: List[int] = []
    for l in layers:
        if used + layer_bytes[l] + arena > budget_bytes:
            break
        resident.append(l)
        used += layer_bytes[l]
    offloaded = [l for l in layers if l not in resident]
    if used + arena > budget_bytes:
        raise MemoryError(f"weight budget of {budget_bytes} bytes cannot hold the resident tensors ({used}) "
                          f"plus a {slots}-slot arena ({arena})")
    return ResidencyPlan(resident, offloaded, layer_bytes, fixed, arena, used + arena,
                         sum(layer_bytes[l] for l in offloaded))


class OffloadedWeights:
    def __init__(self, weights: Dict[str, object], device, budget_bytes: int, prefix: str = "text", slots: int = 2):
        self.device = torch.device(device)
        self.prefix, self.slots = prefix, max(2, slots)
        self.plan = plan_residency(weights, budget_bytes, prefix, self.slots)
        self._resident: Dict[str, object] = {}
        self._host: Dict[int, torch.Tensor] = {}              # layer -> pinned byte image
        self._layout: Dict[int, Dict[str, Tuple[int, tuple, torch.dtype]]] = {}
        off_set = set(self.plan.offloaded_layers)
        per_layer: Dict[int, List[Tuple[str, torch.Tensor]]] = {}
        for name, t in weights.items():
            l = _layer_of(name, prefix)
            if l is None or l not in off_set or not _movable(t):
                self._resident[name] = t.to(self.device) if isinstance(t, torch.Tensor) else t
            else:
                per_layer.setdefault(l, []).append((name, t))
        slot_bytes = 0
        for l, items in per_layer.items():
            off, lay = 0, {}
            for name, t in items:
                off = (off + 255) // 256 * 256
                lay[name] = (off, tuple(t.shape), t.dtype)
                off += t.numel() * t.element_size()
            img = torch.empty(off, dtype=torch.uint8, pin_memory=self.device.type == "cuda")
            for name, t in items:
                o, _, _ = lay[name]
                n = t.numel() * t.element_size()
                img[o:o + n] = t.detach().contiguous().cpu().view(torch.uint8).reshape(-1)
            self._host[l], self._layout[l] = img, lay
            slot_bytes = max(slot_bytes, off)
        self._order = self.plan.offloaded_layers
        self._slot_of = {l: i % self.slots for i, l in enumerate(self._order)}
        self._arena = [torch.empty(slot_bytes, dtype=torch.uint8, device=self.device) for _ in range(self.slots if self._order else 0)]
        self._in_slot: List[Optional[int]] = [None] * len(self._arena)
        self._ready: Dict[int, torch.cuda.Event] = {}
        self._copy = torch.cuda.Stream(device=self.device) if (self._order and self.device.type == "cuda") else None
        self.fetches = 0
        if self._order:
            self._fetch(self._order[0])

    # ---------------------------------------------------------------- mapping interface
    def __contains__(self, name: str) -> bool:
        l = _layer_of(name, self.prefix)
        return name in self._resident or (l in self._layout and name in self._layout[l])

    def __getitem__(self, name: str):
        t = self._resident.get(name)
        if t is not None:
            return t
        l = _layer_of(name, self.prefix)
        if l is None or l not in self._layout or name not in self._layout[l]:
            raise KeyError(name)
        self._ensure(l)
        off, shape, dt = self._layout[l][name]
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dt).element_size()
        return self._arena[self._slot_of[l]][off:off + nbytes].view(dt).view(shape)

    def get(self, name: str, default=None):
        return self[name] if name in self else default

    def keys(self) -> Iterator[str]:
        yield from self._resident
        for lay in self._layout.values():
            yield from lay

    def items(self):
        return ((k, self[k]) for k in self.keys())

    def values(self):
        """Resident objects as they are; offloaded tensors as views of their pinned host image (no fetch)."""
        yield from self._resident.values()
        for l, lay in self._layout.items():
            for off, shape, dt in lay.values():
                n = 1
                for s_ in shape:
                    n *= s_
                yield self._host[l][off:off + n * torch.empty(0, dtype=dt).element_size()].view(dt).view(shape)

    # ---------------------------------------------------------------- rotation
    def _fetch(self, layer: int) -> None:
        slot = self._slot_of[layer]
        if self._in_slot[slot] == layer:
            return
        img = self._host[layer]
        if self._copy is None:
            self._arena[slot][: img.numel()].copy_(img)
        else:
            # the slot's previous tenant may still be read by kernels already enqueued on the compute stream
            self._copy.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._copy):
                self._arena[slot][: img.numel()].copy_(img, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._copy)
            self._ready[layer] = ev
        self._in_slot[slot] = layer
        self.fetches += 1

    def _ensure(self, layer: int) -> None:
        self._fetch(layer)
        ev = self._ready.pop(layer, None)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    def note_layer(self, layer: int) -> None:
        """The forward pass is about to run `layer`: make it available and start bringing in the offloaded layer
        that follows it (cyclically, so the first offloaded layer of the next step is on its way during the head)."""
        if not self._order:
            return
        if layer in self._slot_of:
            self._ensure(layer)
            nxt = self._order[(self._order.index(layer) + 1) % len(self._order)]
        else:
            later = [l for l in self._order if l > layer]
            nxt = later[0] if later else self._order[0]
        if nxt != layer:
            self._fetch(nxt)
