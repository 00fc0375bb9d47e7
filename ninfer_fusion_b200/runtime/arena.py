"""Bump arena over one preallocated device buffer, with scopes and a peak trace.

`alloc` hands out aligned views of the buffer and moves a cursor; `scope()` remembers the cursor and puts it back on
exit, so temporaries of a phase (a layer, a proposal pass) reuse the same bytes as the next phase's; `peak` / `trace`
say how far the cursor ever got and which labelled allocations were live at that moment, which is how the arena's
size is chosen.  Nothing is ever freed individually and nothing allocates after construction, so addresses are
stable across CUDA-graph replays as long as the same sequence of allocations is made.

Counterpart of the reference's DeviceArena / WorkspaceArena scopes (src/core/arena.h:42-81).
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import List, Sequence, Tuple

import torch


class ArenaOverflow(MemoryError):
    pass


class BumpArena:
    def __init__(self, nbytes: int, device, align: int = 256):
        if align & (align - 1):
            raise ValueError("alignment must be a power of two")
        self.buf = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        self.align = align
        self.cursor = 0
        self.peak = 0
        self._live: List[Tuple[str, int, int]] = []       # (label, offset, bytes) of the allocations below the cursor
        self.trace: List[Tuple[str, int, int]] = []       # the live list at the moment of the peak
        # the base address may be less aligned than `align`: offsets are aligned relative to the address
        self._base = self.buf.data_ptr() if self.buf.numel() else 0

    @property
    def capacity(self) -> int:
        return self.buf.numel()

    def alloc(self, shape: Sequence[int], dtype: torch.dtype, label: str = "") -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = ((self._base + self.cursor + self.align - 1) & ~(self.align - 1)) - self._base
        if start + nbytes > self.capacity:
            raise ArenaOverflow(f"arena of {self.capacity} bytes cannot hold '{label or 'allocation'}' of {nbytes} bytes at "
                                f"offset {start} (live: {', '.join(f'{l}:{b}' for l, _, b in self._live) or 'nothing'})")
        self.cursor = start + nbytes
        self._live.append((label, start, nbytes))
        if self.cursor > self.peak:
            self.peak = self.cursor
            self.trace = list(self._live)
        return self.buf[start:start + nbytes].view(dtype).view(*shape)

    @contextmanager
    def scope(self):
        """Everything allocated inside the scope is given back when it ends."""
        mark, n_live = self.cursor, len(self._live)
        try:
            yield self
        finally:
            self.cursor = mark
            del self._live[n_live:]

    def reset(self) -> None:
        self.cursor = 0
        self._live.clear()

    def report(self) -> str:
        rows = "\n".join(f"  {off:>12d}  {nbytes:>12d}  {label}" for label, off, nbytes in self.trace)
        return f"arena {self.capacity} bytes, peak {self.peak} ({100.0 * self.peak / max(1, self.capacity):.1f} %)\n{rows}"
