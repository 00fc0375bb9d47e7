"""Paged KV cache and GDN state pools.

One page id addresses the same token range in every full-attention layer; each
layer owns its planes and may use its own codec (bf16 / fp8-row / int8-group /
nvfp4), which is what per-layer KV policies select.  Page size and the int8
group are parameters (the reference fixes P = 64 and G = 64,
src/core/paged_kv_cache.h:17).  Block tables are an int32 matrix
``[rows, max_pages]`` mirrored in pinned host memory so a decode round uploads
only what changed.

The GDN pools hold, per linear-attention layer, the 3-column conv history and
the fp32 recurrent state per sequence slot (reference:
src/core/linear_attention_state.{h,cpp}; 2C slots = current + turn checkpoint).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..models.config import ModelConfig
from ..ops.reference import KV_BF16, KV_FORMAT_NAMES, KV_FP8_ROW, KV_INT8_GROUP, KV_NVFP4


def kv_row_bytes(fmt: int, head_dim: int) -> int:
    return 2 * head_dim if fmt == KV_BF16 else (head_dim // 2 if fmt == KV_NVFP4 else head_dim)


def kv_scale_bytes(fmt: int, head_dim: int, group: int) -> int:
    if fmt == KV_FP8_ROW:
        return 2
    if fmt == KV_INT8_GROUP:
        return 2 * (head_dim // group)
    if fmt == KV_NVFP4:
        return head_dim // 16
    return 0


@dataclass
class KvLayerPlanes:
    fmt: int
    group: int
    k_codes: torch.Tensor
    v_codes: torch.Tensor
    k_scales: Optional[torch.Tensor]
    v_scales: Optional[torch.Tensor]
    hadamard: bool = False   # K (and the matching Q) live in the normalised Hadamard frame ("fp8h")
    # set when this layer's pages are addressed through ANOTHER cache's block table (a model whose sliding-window
    # layers live in a CyclicKvCache while its other layers live in a full cache); None = the owning cache's table
    block_table: Optional[torch.Tensor] = None

    def bytes(self) -> int:
        n = self.k_codes.numel() + self.v_codes.numel()
        if self.k_scales is not None:
            n += self.k_scales.numel() + self.v_scales.numel()
        return n


KV_MIXED = 4                                   # csrc/kv/kv_layout.h kKvMixed
TIER_FORMATS = (KV_BF16, KV_FP8_ROW, KV_NVFP4)   # tier 0, 1, 2 of a mixed layer
TIER_NAMES = ("bf16", "fp8", "nvfp4")
CELL_TIER_SHIFT = 28


class MixedKvPlanes(KvLayerPlanes):
    """A full-attention layer whose (64-token block x layer) cells live in one of three tiers of falling precision:
    tier 0 bf16, tier 1 fp8-row, tier 2 nvfp4.  Every tier has its own planes and slot allocator; `cell_map[page]`
    (tier << 28 | slot, -1 = none) says where the cell of a logical page is.  New pages start in `hot_tier`; cells
    descend one rung at a time (`PagedKvCache.descend`), which frees a wide slot for a narrow one: that is where
    per-cell precision descent saves device memory.  The attention and append kernels follow the map (format 4).
    Reference: the cell contract of src/product/kv_block_descent.h:1-58 and the narrow sentinels in the block-table
    entries of src/core/paged_kv_cache.h."""

    def __init__(self, n_pages: int, n_kv_heads: int, page_size: int, head_dim: int, device, capacity, hot_tier: int):
        if head_dim != 256:
            raise ValueError("mixed-precision KV layers need head_dim 256")
        self.tiers: List[KvLayerPlanes] = []
        for t, slots in enumerate(capacity):
            fmt = TIER_FORMATS[t]
            group = 16 if fmt == KV_NVFP4 else head_dim
            rb, sb = kv_row_bytes(fmt, head_dim), kv_scale_bytes(fmt, head_dim, group)
            n = max(1, int(slots))
            k = torch.zeros((n, n_kv_heads, page_size, rb), dtype=torch.uint8, device=device)
            v = torch.zeros_like(k)
            ks = vs = None
            if sb:
                ks = torch.zeros((n, n_kv_heads, page_size, sb), dtype=torch.uint8, device=device)
                vs = torch.zeros_like(ks)
            self.tiers.append(KvLayerPlanes(fmt, group, k, v, ks, vs))
        hot = self.tiers[0]
        super().__init__(KV_MIXED, head_dim, hot.k_codes, hot.v_codes, None, None, False)
        self.capacity = [int(c) for c in capacity]
        self.free: List[List[int]] = [list(range(int(c) - 1, -1, -1)) for c in capacity]
        self.hot_tier = hot_tier
        pin = torch.device(device).type == "cuda"
        self.cell_map_host = torch.full((n_pages,), -1, dtype=torch.int32, pin_memory=pin)
        self.cell_map = torch.full((n_pages,), -1, dtype=torch.int32, device=device)
        self.dirty = False
        addr = [self.cell_map.data_ptr()]
        for t in self.tiers:
            addr += [t.k_codes.data_ptr(), t.v_codes.data_ptr(),
                     0 if t.k_scales is None else t.k_scales.data_ptr(), 0 if t.v_scales is None else t.v_scales.data_ptr()]
        self.desc = torch.tensor(addr, dtype=torch.int64)   # what the kernels' bindings read (CPU tensor of addresses)
        self.cell_bytes = [2 * n_kv_heads * page_size * (kv_row_bytes(f, head_dim) +
                                                         kv_scale_bytes(f, head_dim, 16 if f == KV_NVFP4 else head_dim))
                           for f in TIER_FORMATS]

    def bytes(self) -> int:
        return sum(t.bytes() for t in self.tiers)

    def bytes_in_use(self) -> int:
        return sum((self.capacity[t] - len(self.free[t])) * self.cell_bytes[t] for t in range(3))

    def tier_of(self, page: int) -> int:
        c = int(self.cell_map_host[page])
        return -1 if c < 0 else c >> CELL_TIER_SHIFT

    def alloc_cell(self, page: int, tier: Optional[int] = None) -> None:
        t = self.hot_tier if tier is None else tier
        if not self.free[t]:
            raise MemoryError(f"mixed KV layer: tier {TIER_NAMES[t]} has no free cell")
        self.cell_map_host[page] = (t << CELL_TIER_SHIFT) | self.free[t].pop()
        self.dirty = True

    def free_cell(self, page: int) -> None:
        c = int(self.cell_map_host[page])
        if c >= 0:
            self.free[c >> CELL_TIER_SHIFT].append(c & ((1 << CELL_TIER_SHIFT) - 1))
            self.cell_map_host[page] = -1
            self.dirty = True

    def copy_cell(self, p_src: int, p_dst: int) -> None:
        """Cell of `p_dst` := a copy of the cell of `p_src`, in the same tier."""
        c = int(self.cell_map_host[p_src])
        t, s_src = c >> CELL_TIER_SHIFT, c & ((1 << CELL_TIER_SHIFT) - 1)
        self.free_cell(p_dst)
        self.alloc_cell(p_dst, t)
        s_dst = int(self.cell_map_host[p_dst]) & ((1 << CELL_TIER_SHIFT) - 1)
        tp = self.tiers[t]
        for plane in (tp.k_codes, tp.v_codes, tp.k_scales, tp.v_scales):
            if plane is not None:
                plane[s_dst].copy_(plane[s_src])

    def publish(self) -> None:
        if self.dirty:
            self.cell_map.copy_(self.cell_map_host, non_blocking=True)
            self.dirty = False


def _load_pool_lib():
    import ctypes
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")
    if not os.path.exists(path):
        return None
    try:
        lib = ctypes.CDLL(path)
        lib.nfb200_pool_create.restype = ctypes.c_void_p
        lib.nfb200_pool_create.argtypes = [ctypes.c_int32]
        lib.nfb200_pool_destroy.argtypes = [ctypes.c_void_p]
        for name in ("free_pages", "alloc"):
            getattr(lib, f"nfb200_pool_{name}").restype = ctypes.c_int32
            getattr(lib, f"nfb200_pool_{name}").argtypes = [ctypes.c_void_p]
        for name in ("retain", "release", "refcount"):
            getattr(lib, f"nfb200_pool_{name}").restype = ctypes.c_int32
            getattr(lib, f"nfb200_pool_{name}").argtypes = [ctypes.c_void_p, ctypes.c_int32]
        return lib
    except (OSError, AttributeError):
        return None


class PagePool:
    """Reference-counted page allocator.  The bookkeeping runs in native code (csrc/runtime/page_pool.cpp) when the
    library is built; the pure-Python twin has the same semantics."""

    def __init__(self, n_pages: int, use_native: bool = True):
        self.n_pages = n_pages
        self._lib = _load_pool_lib() if use_native else None
        self._h = self._lib.nfb200_pool_create(n_pages) if self._lib is not None else None
        if self._h is None:
            self._free: List[int] = list(range(n_pages - 1, -1, -1))
            self._ref = [0] * n_pages

    def __del__(self):
        if getattr(self, "_h", None) is not None:
            self._lib.nfb200_pool_destroy(self._h)
            self._h = None

    @property
    def native(self) -> bool:
        return self._h is not None

    @property
    def free_pages(self) -> int:
        return int(self._lib.nfb200_pool_free_pages(self._h)) if self._h is not None else len(self._free)

    def refcount_of(self, page: int) -> int:
        return int(self._lib.nfb200_pool_refcount(self._h, page)) if self._h is not None else self._ref[page]

    def alloc(self) -> int:
        if self._h is not None:
            p = int(self._lib.nfb200_pool_alloc(self._h))
            if p < 0:
                raise MemoryError("KV page pool exhausted")
            return p
        if not self._free:
            raise MemoryError("KV page pool exhausted")
        p = self._free.pop()
        self._ref[p] = 1
        return p

    def retain(self, page: int) -> None:
        if self._h is not None:
            if self._lib.nfb200_pool_retain(self._h, page) < 0:
                raise RuntimeError(f"page {page} is not allocated")
            return
        if self._ref[page] <= 0:
            raise RuntimeError(f"page {page} is not allocated")
        self._ref[page] += 1

    def release(self, page: int) -> None:
        if self._h is not None:
            if self._lib.nfb200_pool_release(self._h, page) < 0:
                raise RuntimeError(f"page {page} released twice")
            return
        if self._ref[page] <= 0:
            raise RuntimeError(f"page {page} released twice")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)


class PagedKvCache:
    def __init__(self, cfg: ModelConfig, n_pages: int, page_size: int, max_rows: int, max_pages_per_row: int,
                 device, formats: Sequence[str] | str = "bf16", int8_group: int = 64,
                 n_kv_heads: Optional[int] = None, n_layers: Optional[int] = None,
                 mixed_capacity: Optional[Sequence[int]] = None, mixed_hot_tier: int = 0):
        """`formats` entry "mixed": that layer keeps its cells in three tiers (MixedKvPlanes); `mixed_capacity` =
        cells per tier (default: every tier can hold every page), `mixed_hot_tier` = where new pages start."""
        self.cfg = cfg
        self.page_size = page_size
        self.n_pages = n_pages
        self.device = torch.device(device)
        self.n_kv_heads = n_kv_heads if n_kv_heads is not None else cfg.n_kv_heads
        n_attn = n_layers if n_layers is not None else len(cfg.attn_layers)
        if isinstance(formats, str):
            formats = [formats] * n_attn
        if len(formats) != n_attn:
            raise ValueError(f"need one KV format per full-attention layer ({n_attn}), got {len(formats)}")
        D = cfg.head_dim
        self.layers: List[KvLayerPlanes] = []
        for name in formats:
            if name == "mixed":
                cap = list(mixed_capacity) if mixed_capacity is not None else [n_pages, n_pages, n_pages]
                self.layers.append(MixedKvPlanes(n_pages, self.n_kv_heads, page_size, D, self.device, cap, mixed_hot_tier))
                continue
            hadamard = name == "fp8h"   # fp8 per-row codec with K stored in the Hadamard frame
            fmt = KV_FORMAT_NAMES["fp8" if hadamard else name]
            group = int8_group if fmt == KV_INT8_GROUP else (16 if fmt == KV_NVFP4 else D)
            rb, sb = kv_row_bytes(fmt, D), kv_scale_bytes(fmt, D, group)
            shape = (n_pages, self.n_kv_heads, page_size, rb)
            k = torch.zeros(shape, dtype=torch.uint8, device=self.device)
            v = torch.zeros(shape, dtype=torch.uint8, device=self.device)
            ks = vs = None
            if sb:
                ks = torch.zeros((n_pages, self.n_kv_heads, page_size, sb), dtype=torch.uint8, device=self.device)
                vs = torch.zeros_like(ks)
            self.layers.append(KvLayerPlanes(fmt, group, k, v, ks, vs, hadamard))
        self.mixed = [l for l in self.layers if isinstance(l, MixedKvPlanes)]
        self.pool = PagePool(n_pages)
        self.host_arena = None   # optional runtime.host_arena.HostKvArena for the cold copies of exported pages
        # Lossy cold copies: int8 group-64 layers leave the device as requantised cold slots (E2M1 codes + E4M3 scales
        # per 16 values, 9232 bytes per 64 x 256 page plane instead of 16896) packed by a device kernel before the
        # D2H copy; a page warmed from its slot is close to, not identical with, the page that was retired.
        self.cold_slots = False
        self.max_rows = max_rows
        self.max_pages_per_row = max_pages_per_row
        pin = self.device.type == "cuda"
        self.table_host = torch.full((max_rows, max_pages_per_row), -1, dtype=torch.int32, pin_memory=pin)
        self.table = torch.full((max_rows, max_pages_per_row), -1, dtype=torch.int32, device=self.device)
        self.row_pages: Dict[int, List[int]] = {}
        self._dirty_rows: set[int] = set()

    # ---- capacity ----
    def bytes_per_token(self) -> float:
        return sum(l.bytes() for l in self.layers) / (self.n_pages * self.page_size)

    def total_bytes(self) -> int:
        return sum(l.bytes() for l in self.layers)

    # ---- logical pages (and, for mixed layers, their cells) ----
    def _page_alloc(self) -> int:
        p = self.pool.alloc()
        try:
            for l in self.mixed:
                l.alloc_cell(p)
        except MemoryError:
            for l in self.mixed:
                l.free_cell(p)
            self.pool.release(p)
            raise
        return p

    def _page_release(self, p: int) -> None:
        self.pool.release(p)
        if self.mixed and self.pool.refcount_of(p) == 0:
            for l in self.mixed:
                l.free_cell(p)

    def bytes_in_use(self) -> int:
        """Device bytes of the cells that hold live pages (mixed layers: by each cell's tier)."""
        used = self.n_pages - self.pool.free_pages
        n = 0
        for l in self.layers:
            n += l.bytes_in_use() if isinstance(l, MixedKvPlanes) else l.bytes() // self.n_pages * used
        return n

    def tier_census(self) -> Dict[str, int]:
        """Cells per tier over all mixed layers."""
        out = {name: 0 for name in TIER_NAMES}
        for l in self.mixed:
            for t, name in enumerate(TIER_NAMES):
                out[name] += l.capacity[t] - len(l.free[t])
        return out

    def descend(self, layer_index: int, pages: Sequence[int], to_tier: int) -> int:
        """Re-encodes the cells of `pages` in mixed layer `layer_index` into `to_tier` (one launch) and frees their old
        slots.  Cells already there, or without a free target slot, are skipped; returns the number moved.  Call
        between steps: the kernel and the map update are ordered on the current stream."""
        l = self.layers[layer_index]
        if not isinstance(l, MixedKvPlanes):
            raise ValueError(f"layer {layer_index} is not a mixed-precision layer")
        src, dst, moved = [], [], []
        for p in pages:
            c = int(l.cell_map_host[p])
            if c < 0 or (c >> CELL_TIER_SHIFT) == to_tier or not l.free[to_tier]:
                continue
            src.append(c)
            dst.append((to_tier << CELL_TIER_SHIFT) | l.free[to_tier].pop())
            moved.append(p)
        if not moved:
            return 0
        from .._lib import load_native
        ops = load_native()
        s = torch.tensor(src, dtype=torch.int32).to(self.device, non_blocking=True)
        d = torch.tensor(dst, dtype=torch.int32).to(self.device, non_blocking=True)
        ops.kv_requant(l.desc, l.tiers[0].k_codes, s, d, self.page_size, self.n_kv_heads, self.cfg.head_dim)
        for p, c_old, c_new in zip(moved, src, dst):
            l.free[c_old >> CELL_TIER_SHIFT].append(c_old & ((1 << CELL_TIER_SHIFT) - 1))
            l.cell_map_host[p] = c_new
        l.dirty = True
        l.publish()
        return len(moved)

    # ---- mapping ----
    def ensure(self, row: int, n_tokens: int) -> None:
        """Make sure `row` has pages for positions [0, n_tokens)."""
        pages = self.row_pages.setdefault(row, [])
        need = (n_tokens + self.page_size - 1) // self.page_size
        if need > self.max_pages_per_row:
            raise MemoryError(f"row {row}: {n_tokens} tokens exceed the block-table width")
        while len(pages) < need:
            p = self._page_alloc()
            self.table_host[row, len(pages)] = p
            pages.append(p)
            self._dirty_rows.add(row)

    def trim(self, row: int, n_tokens: int) -> None:
        """Drop pages that lie wholly beyond n_tokens (speculative rollback)."""
        pages = self.row_pages.get(row, [])
        keep = (n_tokens + self.page_size - 1) // self.page_size
        while len(pages) > keep:
            p = pages.pop()
            self.table_host[row, len(pages)] = -1
            if p >= 0:
                self._page_release(p)
            self._dirty_rows.add(row)

    def release_before(self, row: int, n_tokens: int, window: int, slack: int = 64) -> int:
        """Sliding-window layers never look further back than `window` keys: pages that lie wholly before
        n_tokens + 1 - window - slack go back to the pool (the row behaves like a ring over a bounded number of
        pages; `slack` covers the prefill kernel's tile rounding).  The freed positions keep their place in the
        block table as -1.  Returns the number of pages released.  Only valid when EVERY layer sharing this table
        is windowed."""
        if window <= 0:
            return 0
        pages = self.row_pages.get(row, [])
        first_needed = max(0, n_tokens + 1 - window - slack)
        n = 0
        for i in range(min(len(pages), first_needed // self.page_size)):
            if pages[i] >= 0:
                self._page_release(pages[i])
                pages[i] = -1
                self.table_host[row, i] = -1
                n += 1
        if n:
            self._dirty_rows.add(row)
        return n

    def free_row(self, row: int) -> None:
        for p in self.row_pages.pop(row, []):
            if p >= 0:
                self._page_release(p)
        self.table_host[row].fill_(-1)
        self._dirty_rows.add(row)

    def fork_row(self, src: int, dst: int, n_tokens: int) -> None:
        """Share src's full pages with dst (prefix reuse); a partial tail page is copied."""
        self.free_row(dst)
        full = n_tokens // self.page_size
        pages = self.row_pages.setdefault(dst, [])
        if any(p < 0 for p in self.row_pages[src][: full + 1]):
            raise ValueError("a row whose early pages were released (sliding window) cannot be forked")
        for i in range(full):
            p = self.row_pages[src][i]
            self.pool.retain(p)
            pages.append(p)
            self.table_host[dst, i] = p
        if n_tokens % self.page_size:
            p_src = self.row_pages[src][full]
            p_new = self._page_alloc()
            self._copy_page(p_src, p_new)
            pages.append(p_new)
            self.table_host[dst, full] = p_new
        self._dirty_rows.add(dst)

    # ---- detached page lists (session checkpoints): they hold page references but own no block-table row ----
    def detach_prefix(self, src_row: int, n_tokens: int) -> Optional[List[int]]:
        """Page list covering positions [0, n_tokens) of `src_row`: full pages are shared (retained), a partial tail
        page is copied so that the source may keep appending into its own.  None if the pool is exhausted."""
        full = n_tokens // self.page_size
        tail = n_tokens % self.page_size
        if tail and self.pool.free_pages < 1:
            return None
        src = self.row_pages[src_row]
        if any(p < 0 for p in src[: full + (1 if tail else 0)]):
            return None   # early pages were released (sliding window): this history cannot become a frontier
        pages = []
        for i in range(full):
            self.pool.retain(src[i])
            pages.append(src[i])
        if tail:
            p_new = self._page_alloc()
            self._copy_page(src[full], p_new)
            pages.append(p_new)
        return pages

    def attach_prefix(self, pages: List[int], dst_row: int, n_tokens: int) -> None:
        """Make `dst_row` start from a detached page list (full pages shared, partial tail page copied)."""
        self.free_row(dst_row)
        full = n_tokens // self.page_size
        mine = self.row_pages.setdefault(dst_row, [])
        for i in range(full):
            self.pool.retain(pages[i])
            mine.append(pages[i])
            self.table_host[dst_row, i] = pages[i]
        if n_tokens % self.page_size:
            p_new = self._page_alloc()
            self._copy_page(pages[full], p_new)
            mine.append(p_new)
            self.table_host[dst_row, full] = p_new
        self._dirty_rows.add(dst_row)

    # ---- cold tiers: page contents leave / re-enter the device pool ----
    def export_pages(self, pages: List[int]) -> List[torch.Tensor]:
        """Contents of `pages` in every layer as pinned host tensors (device -> host, D2H page copies)."""
        if self.mixed:
            raise NotImplementedError("cold copies of mixed-precision layers are not built: their cells already descend")
        idx = torch.tensor(pages, dtype=torch.long, device=self.device)
        out = []
        pin = self.device.type == "cuda"
        for l in self.layers:
            if self._slot_layer(l):
                from .._lib import load_native
                ops = load_native()
                D = self.cfg.head_dim
                for codes, scales in ((l.k_codes, l.k_scales), (l.v_codes, l.v_scales)):
                    c = codes.index_select(0, idx).view(torch.int8).reshape(-1, D)
                    sc = scales.index_select(0, idx).view(torch.float16).reshape(-1, D // 64)
                    dev = ops.cold_slot_pack_int8(c, sc, self.page_size)      # [pages * heads, slot bytes]
                    host = torch.empty(dev.shape, dtype=dev.dtype, pin_memory=pin)
                    host.copy_(dev, non_blocking=True)
                    out.append(host)
                continue
            for plane in (l.k_codes, l.v_codes, l.k_scales, l.v_scales):
                if plane is None:
                    continue
                dev = plane.index_select(0, idx)
                host = self.host_arena.alloc_like(dev) if self.host_arena is not None else None
                if host is None:   # no arena, or no free run large enough: a private pinned allocation
                    host = torch.empty(dev.shape, dtype=dev.dtype, pin_memory=pin)
                host.copy_(dev, non_blocking=True)
                out.append(host)
        if pin:
            torch.cuda.current_stream(self.device).synchronize()
        return out

    def import_pages(self, planes: List[torch.Tensor], n_pages: int) -> Optional[List[int]]:
        """Allocates `n_pages` fresh pages and fills them from `export_pages` output.  None if the pool is too small."""
        if self.pool.free_pages < n_pages:
            return None
        pages = [self._page_alloc() for _ in range(n_pages)]
        idx = torch.tensor(pages, dtype=torch.long, device=self.device)
        it = iter(planes)
        for l in self.layers:
            if self._slot_layer(l):
                from .._lib import load_native
                ops = load_native()
                D = self.cfg.head_dim
                for codes, scales in ((l.k_codes, l.k_scales), (l.v_codes, l.v_scales)):
                    slots = next(it).to(self.device, non_blocking=True)
                    c, sc = ops.cold_slot_restore_int8(slots, self.page_size, D)
                    codes.index_copy_(0, idx, c.view(torch.uint8).reshape(n_pages, self.n_kv_heads, self.page_size, D))
                    scales.index_copy_(0, idx, sc.view(torch.uint8).reshape(n_pages, self.n_kv_heads, self.page_size, -1))
                continue
            for plane in (l.k_codes, l.v_codes, l.k_scales, l.v_scales):
                if plane is None:
                    continue
                plane.index_copy_(0, idx, next(it).to(self.device, non_blocking=True))
        return pages

    def _slot_layer(self, l: "KvLayerPlanes") -> bool:
        """A layer whose cold copies are requantised slots: lossy copies switched on, int8 with 64-value groups, on a GPU."""
        return (self.cold_slots and l.fmt == KV_INT8_GROUP and l.group == 64 and self.cfg.head_dim % 64 == 0
                and self.device.type == "cuda")

    def drop_pages(self, pages: List[int]) -> None:
        for p in pages:
            self._page_release(p)

    def _copy_page(self, p_src: int, p_dst: int) -> None:
        for l in self.layers:
            if isinstance(l, MixedKvPlanes):
                l.copy_cell(p_src, p_dst)
                continue
            l.k_codes[p_dst].copy_(l.k_codes[p_src])
            l.v_codes[p_dst].copy_(l.v_codes[p_src])
            if l.k_scales is not None:
                l.k_scales[p_dst].copy_(l.k_scales[p_src])
                l.v_scales[p_dst].copy_(l.v_scales[p_src])

    def publish(self) -> None:
        """Upload dirty block-table rows (and the cell maps of mixed layers) to the device."""
        for l in self.mixed:
            l.publish()
        if not self._dirty_rows:
            return
        if len(self._dirty_rows) > 8:
            self.table.copy_(self.table_host, non_blocking=True)
        else:
            for r in self._dirty_rows:
                self.table[r].copy_(self.table_host[r], non_blocking=True)
        self._dirty_rows.clear()


class CyclicKvCache(PagedKvCache):
    """KV cache of sliding-window layers: every row owns a bounded ring of pages however long the sequence grows.

    A windowed layer never looks further back than `window` keys, so a row needs pages for window + slack + one
    page of positions only.  The block table keeps one entry per logical page of the whole context (so the kernels
    address it exactly like a full cache); `ensure` first returns the pages that slid out of the window to the pool
    (their table entries become -1: the attention kernels skip such pages) and then maps the new positions, which
    reuses those physical pages.  Only valid when EVERY layer of this cache is windowed.

    Counterpart of the reference's cyclic cache for its sliding-window / DFlash local layers
    (src/core/cyclic_kv_cache.h); here the ring is a property of the page map, not a second kernel interface."""

    def __init__(self, cfg: ModelConfig, window: int, page_size: int, max_rows: int, max_context: int, device,
                 formats: Sequence[str] | str = "bf16", slack: int = 64, n_kv_heads: Optional[int] = None,
                 n_layers: Optional[int] = None):
        if window <= 0:
            raise ValueError("a cyclic cache needs a positive window")
        self.window, self.slack = window, slack
        self.ring_pages = (window + slack + page_size - 1) // page_size + 2   # + the partial pages at both ends
        super().__init__(cfg, max_rows * self.ring_pages, page_size, max_rows, (max_context + page_size - 1) // page_size,
                         device, formats=formats, n_kv_heads=n_kv_heads, n_layers=n_layers)

    def ensure(self, row: int, n_tokens: int) -> None:
        self.release_before(row, n_tokens, self.window, self.slack)
        pages = self.row_pages.setdefault(row, [])
        need = (n_tokens + self.page_size - 1) // self.page_size
        if need > self.max_pages_per_row:
            raise MemoryError(f"row {row}: {n_tokens} tokens exceed the block-table width")
        # positions before the window that were never mapped stay unmapped
        first_needed = max(0, n_tokens + 1 - self.window - self.slack) // self.page_size
        while len(pages) < min(first_needed, need):
            pages.append(-1)
        while len(pages) < need:
            p = self._page_alloc()
            self.table_host[row, len(pages)] = p
            pages.append(p)
            self._dirty_rows.add(row)

    def live_pages(self, row: int) -> int:
        return sum(1 for p in self.row_pages.get(row, []) if p >= 0)


class GdnStatePool:
    """Conv history + fp32 recurrent state for every GDN layer, `n_slots` sequence slots."""

    def __init__(self, cfg: ModelConfig, n_slots: int, device, n_qk_heads: Optional[int] = None,
                 n_v_heads: Optional[int] = None, n_layers: Optional[int] = None):
        self.cfg = cfg
        self.n_slots = n_slots
        hk = n_qk_heads if n_qk_heads is not None else cfg.gdn_qk_heads
        hv = n_v_heads if n_v_heads is not None else cfg.gdn_v_heads
        n_gdn = n_layers if n_layers is not None else len(cfg.gdn_layers)
        d = cfg.gdn_head_dim
        self.conv_dim = (2 * hk + hv) * d
        self.conv = [torch.zeros((n_slots, 3, self.conv_dim), dtype=torch.bfloat16, device=device)
                     for _ in range(n_gdn)]
        self.ssm = [torch.zeros((n_slots, hv, d, d), dtype=torch.float32, device=device) for _ in range(n_gdn)]
        self._free = list(range(n_slots - 1, -1, -1))

    def alloc(self) -> int:
        if not self._free:
            raise MemoryError("GDN state slots exhausted")
        s = self._free.pop()
        self.reset(s)
        return s

    def release(self, slot: int) -> None:
        self._free.append(slot)

    def reset(self, slot: int) -> None:
        for c, s in zip(self.conv, self.ssm):
            c[slot].zero_()
            s[slot].zero_()

    def copy_slot(self, src: int, dst: int) -> None:
        """Checkpoint / fork a sequence's recurrent state."""
        for c, s in zip(self.conv, self.ssm):
            c[dst].copy_(c[src])
            s[dst].copy_(s[src])

    def export_slot(self, slot: int) -> List[torch.Tensor]:
        """State image of one slot (conv history + recurrent state of every layer) as pinned host tensors."""
        pin = self.conv[0].device.type == "cuda"
        out = []
        for c, s in zip(self.conv, self.ssm):
            for t in (c[slot], s[slot]):
                host = torch.empty(t.shape, dtype=t.dtype, pin_memory=pin)
                host.copy_(t, non_blocking=True)
                out.append(host)
        if pin:
            torch.cuda.current_stream(self.conv[0].device).synchronize()
        return out

    def import_slot(self, image: List[torch.Tensor], slot: int) -> None:
        it = iter(image)
        for c, s in zip(self.conv, self.ssm):
            c[slot].copy_(next(it), non_blocking=True)
            s[slot].copy_(next(it), non_blocking=True)

    def total_bytes(self) -> int:
        return sum(c.numel() * 2 + s.numel() * 4 for c, s in zip(self.conv, self.ssm))
