"""Startup-fixed pinned host arena for cold KV replicas and state images.

One pinned buffer is allocated when the engine starts (pinning is expensive and fragments the host address space when
done per checkpoint); extents inside it are handed out by a first-fit allocator with coalescing.  The bookkeeping
runs in native code (csrc/runtime/host_arena.cpp) when the library is built; the pure-Python twin has the same
semantics.  Reference: src/core/host_kv_arena.{h,cpp}.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from typing import Dict, List, Optional, Tuple

import torch

GRANULE = 256


def _load_lib():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")
    if not os.path.exists(path):
        return None
    try:
        lib = ctypes.CDLL(path)
        lib.nfb200_arena_create.restype = ctypes.c_void_p
        lib.nfb200_arena_create.argtypes = [ctypes.c_int64]
        lib.nfb200_arena_destroy.argtypes = [ctypes.c_void_p]
        lib.nfb200_arena_alloc.restype = ctypes.c_int64
        lib.nfb200_arena_alloc.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_uint32)]
        lib.nfb200_arena_free.restype = ctypes.c_int32
        lib.nfb200_arena_free.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint32]
        for name in ("used", "peak", "capacity", "largest_free"):
            getattr(lib, f"nfb200_arena_{name}").restype = ctypes.c_int64
            getattr(lib, f"nfb200_arena_{name}").argtypes = [ctypes.c_void_p]
        lib.nfb200_arena_live_extents.restype = ctypes.c_int32
        lib.nfb200_arena_live_extents.argtypes = [ctypes.c_void_p]
        return lib
    except (OSError, AttributeError):
        return None


class _PyArena:
    def __init__(self, capacity: int):
        self.capacity = capacity // GRANULE * GRANULE
        self.free: Dict[int, int] = {0: self.capacity} if self.capacity else {}
        self.live: Dict[int, Tuple[int, int]] = {}
        self.used = self.peak = 0
        self.gen = 1

    def alloc(self, nbytes: int):
        need = (nbytes + GRANULE - 1) // GRANULE * GRANULE
        for off in sorted(self.free):
            run = self.free[off]
            if run >= need:
                del self.free[off]
                if run > need:
                    self.free[off + need] = run - need
                g, self.gen = self.gen, self.gen + 1
                self.live[off] = (need, g)
                self.used += need
                self.peak = max(self.peak, self.used)
                return off, g
        return -1, 0

    def free_extent(self, off: int, gen: int) -> int:
        e = self.live.get(off)
        if e is None or e[1] != gen:
            return -1
        run = e[0]
        del self.live[off]
        self.used -= run
        if off + run in self.free:
            run += self.free.pop(off + run)
        for o in list(self.free):
            if o + self.free[o] == off:
                off, run = o, run + self.free.pop(o)
                break
        self.free[off] = run
        return 0


class HostKvArena:
    """`alloc(nbytes)` -> (handle, uint8 tensor view into the pinned buffer) or None when no run is large enough."""

    def __init__(self, capacity_bytes: int, pin: Optional[bool] = None, use_native: bool = True):
        pin = torch.cuda.is_available() if pin is None else pin
        self.buffer = torch.empty(capacity_bytes // GRANULE * GRANULE, dtype=torch.uint8, pin_memory=pin)
        self._lib = _load_lib() if use_native else None
        self._h = self._lib.nfb200_arena_create(self.buffer.numel()) if self._lib is not None else None
        self._py = _PyArena(self.buffer.numel()) if self._h is None else None

    def __del__(self):
        if getattr(self, "_h", None) is not None:
            self._lib.nfb200_arena_destroy(self._h)
            self._h = None

    @property
    def native(self) -> bool:
        return self._h is not None

    def alloc(self, nbytes: int):
        if nbytes <= 0:
            raise ValueError("extent size must be positive")
        if self._h is not None:
            gen = ctypes.c_uint32(0)
            off = int(self._lib.nfb200_arena_alloc(self._h, nbytes, ctypes.byref(gen)))
            g = int(gen.value)
        else:
            off, g = self._py.alloc(nbytes)
        if off < 0:
            return None
        return (off, g), self.buffer[off:off + nbytes]

    def free(self, handle) -> None:
        off, g = handle
        rc = self._lib.nfb200_arena_free(self._h, off, g) if self._h is not None else self._py.free_extent(off, g)
        if rc != 0:
            raise RuntimeError(f"host arena: extent ({off}, generation {g}) is not live")

    def alloc_like(self, t: torch.Tensor) -> Optional[torch.Tensor]:
        """A tensor of t's shape and dtype inside the arena, released when the returned tensor is garbage collected."""
        got = self.alloc(t.numel() * t.element_size())
        if got is None:
            return None
        handle, raw = got
        view = raw.view(t.dtype).view(t.shape)
        weakref.finalize(view, self._free_quiet, handle)
        return view

    def _free_quiet(self, handle) -> None:
        try:
            self.free(handle)
        except RuntimeError:
            pass

    def _stat(self, name: str) -> int:
        if self._h is not None:
            return int(getattr(self._lib, f"nfb200_arena_{name}")(self._h))
        return {"used": self._py.used, "peak": self._py.peak, "capacity": self._py.capacity,
                "largest_free": max(self._py.free.values(), default=0), "live_extents": len(self._py.live)}[name]

    @property
    def used(self) -> int:
        return self._stat("used")

    @property
    def peak(self) -> int:
        return self._stat("peak")

    @property
    def capacity(self) -> int:
        return self._stat("capacity")

    @property
    def largest_free(self) -> int:
        return self._stat("largest_free")

    @property
    def live_extents(self) -> int:
        return self._stat("live_extents")
