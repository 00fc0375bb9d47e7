"""KV capacity: how many physical pages the main pool gets.

With S = max_context, C = max_concurrency, P = page size and L = ceil(S / P) logical pages per sequence, the pool may
hold between M_min = max(L, C) pages (one request can reach S and every lane can hold a page) and M_max = C * L (all
lanes at the ceiling).  An explicit capacity is a token count K >= S giving M = ceil(K / P) inside that range.  The
automatic policy is resolved once after the weights are on the device: the layout builder provides the affine curve
B(M) = B_min + (M - M_min) * B_step (bytes the runtime reserves for a pool of M pages: KV planes, recurrent state
slots, block tables, workspace, a CUDA-graph allowance) and M = min(M_max, M_min + floor((F - R - B_min) / B_step))
for F free bytes and R bytes of headroom; F < R + B_min is refused.  Nothing is probed by allocation.

Reference: src/runtime/engine/kv_capacity.cpp, docs/maintainer/paged-kv-cache.md:87-153.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Union

from ..models.config import ModelConfig


class CapacityError(ValueError):
    pass


@dataclass(frozen=True)
class CapacityCurve:
    m_min: int
    m_max: int
    b_min: int       # bytes reserved at m_min pages
    b_step: int      # bytes per additional page

    def bytes_at(self, pages: int) -> int:
        return self.b_min + (pages - self.m_min) * self.b_step


@dataclass(frozen=True)
class CapacityPlan:
    pages: int
    tokens: int            # pages * page_size: the public "main KV capacity" in token equivalents
    reserved_bytes: int
    policy: str            # "explicit" | "auto" | "full"


def page_range(max_context: int, max_concurrency: int, page_size: int):
    if max_context <= 0 or max_concurrency <= 0 or page_size <= 0:
        raise CapacityError("max_context, max_concurrency and page_size must be positive")
    L = -(-max_context // page_size)
    return max(L, max_concurrency), max_concurrency * L


def kv_page_bytes(cfg: ModelConfig, formats: Union[str, Sequence[str]], page_size: int, n_kv_heads: Optional[int] = None,
                  int8_group: int = 64) -> int:
    """Bytes one physical page takes over all attention layers (K and V codes + their scales), from the same row
    geometry the cache allocates with."""
    from .kv_cache import KV_FORMAT_NAMES, kv_row_bytes, kv_scale_bytes
    names = [formats] * len(cfg.attn_layers) if isinstance(formats, str) else list(formats)
    if len(names) != len(cfg.attn_layers):
        raise CapacityError(f"{len(names)} KV formats for {len(cfg.attn_layers)} attention layers")
    H = cfg.n_kv_heads if n_kv_heads is None else n_kv_heads
    total = 0
    for name in names:
        fmt = KV_FORMAT_NAMES["fp8" if name == "fp8h" else name]
        group = int8_group if name == "int8" else 16
        total += 2 * H * page_size * (kv_row_bytes(fmt, cfg.head_dim) + kv_scale_bytes(fmt, cfg.head_dim, group))
    return total


def build_curve(cfg: ModelConfig, formats, page_size: int, max_context: int, max_concurrency: int,
                checkpoint_slots: Optional[int] = None, workspace_bytes: int = 0, graph_allowance_bytes: int = 256 << 20,
                n_kv_heads: Optional[int] = None, gdn_v_heads: Optional[int] = None) -> CapacityCurve:
    m_min, m_max = page_range(max_context, max_concurrency, page_size)
    step = kv_page_bytes(cfg, formats, page_size, n_kv_heads)
    slots = max_concurrency + (max_concurrency if checkpoint_slots is None else checkpoint_slots)
    hv = cfg.gdn_v_heads if gdn_v_heads is None else gdn_v_heads
    d = cfg.gdn_head_dim
    state = len(cfg.gdn_layers) * slots * (hv * d * d * 4 + 3 * cfg.gdn_conv_dim * 2)      # fp32 state + bf16 conv taps
    L = -(-max_context // page_size)
    tables = max_concurrency * L * 4
    fixed = state + tables + workspace_bytes + graph_allowance_bytes
    return CapacityCurve(m_min, m_max, fixed + m_min * step, step)


def resolve(curve: CapacityCurve, page_size: int, max_context: int, explicit_tokens: Optional[int] = None,
            free_bytes: Optional[int] = None, headroom_bytes: int = 0) -> CapacityPlan:
    """explicit_tokens: the explicit policy; else free_bytes: the automatic policy; neither: the full pool M_max."""
    if explicit_tokens is not None:
        if explicit_tokens < max_context:
            raise CapacityError(f"kv capacity {explicit_tokens} is below max_context {max_context}")
        pages = -(-explicit_tokens // page_size)
        if not curve.m_min <= pages <= curve.m_max:
            raise CapacityError(f"kv capacity of {pages} pages is outside [{curve.m_min}, {curve.m_max}]")
        return CapacityPlan(pages, pages * page_size, curve.bytes_at(pages), "explicit")
    if free_bytes is None:
        return CapacityPlan(curve.m_max, curve.m_max * page_size, curve.bytes_at(curve.m_max), "full")
    if free_bytes < headroom_bytes + curve.b_min:
        raise CapacityError(f"{free_bytes} free bytes cannot hold the minimum reservation {curve.b_min} plus "
                            f"{headroom_bytes} of headroom")
    if curve.m_min == curve.m_max:
        pages = curve.m_min
    else:
        pages = min(curve.m_max, curve.m_min + (free_bytes - headroom_bytes - curve.b_min) // curve.b_step)
    return CapacityPlan(pages, pages * page_size, curve.bytes_at(pages), "auto")
