"""Device memory behind the cache manager's page ids and state slots.

One tensor per group, `[caches of the group, 2 (keys, values), pages, kv heads,
page_size, head_dim]`: for one kv head the `page_size` keys of a page are
contiguous rows of `head_dim` elements, which is the tile an attention kernel
loads.  Per-request state of fixed size lives in one tensor per cache that asks
for it, `[slots, *shape]`.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .manager import CacheManager, GroupKey, Window


@dataclass(frozen=True)
class PagedKV:
    """A mixer's request for paged keys and values."""
    window: Window
    num_kv_heads: int
    head_dim: int


@dataclass(frozen=True)
class FixedState:
    """A mixer's request for per-request state of fixed size."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class LayerCache:
    """What one run of a layer sees of the cache."""

    def __init__(self, group: int | None, kv: torch.Tensor | None, state: torch.Tensor | None,
                 page_size: int, write: bool):
        self.group = group          # index of the block table to use
        self.kv = kv                # [2, pages, kv heads, page_size, head_dim] or None
        self.state = state          # [slots, *shape] or None
        self.page_size = page_size
        self.write = write          # this run appends its keys and values


class CacheStorage:
    def __init__(self, cache_specs: dict, page_size: int, pages: int, n_slots: int,
                 dtype: torch.dtype, device):
        """`cache_specs[cache id] = (PagedKV | None, FixedState | None)`."""
        self.page_size = page_size
        self.device = torch.device(device)
        self.dtype = dtype
        keys: list[GroupKey] = []
        self._group_of = {}
        self._index_in_group = {}
        counts = []
        for cid in sorted(cache_specs):
            kv, _ = cache_specs[cid]
            if kv is None:
                continue
            key = GroupKey(kv.window, kv.num_kv_heads, kv.head_dim)
            if key not in keys:
                keys.append(key)
                counts.append(0)
            g = keys.index(key)
            self._group_of[cid] = g
            self._index_in_group[cid] = counts[g]
            counts[g] += 1
        self.group_keys = keys
        self.manager = CacheManager(keys, page_size, pages if keys else 1, n_slots) if keys else \
            CacheManager([], page_size, [], n_slots)
        self.kv = [torch.zeros((counts[g], 2, pages, k.num_kv_heads, page_size, k.head_dim),
                               dtype=dtype, device=self.device) for g, k in enumerate(keys)]
        self.state = {}
        for cid, (_, st) in cache_specs.items():
            if st is not None:
                self.state[cid] = torch.zeros((n_slots,) + tuple(st.shape), dtype=st.dtype, device=self.device)

    @property
    def n_groups(self):
        return len(self.group_keys)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.state.values())

    def layer_cache(self, cache_id: int, write: bool) -> LayerCache:
        g = self._group_of.get(cache_id)
        kv = self.kv[g][self._index_in_group[cache_id]] if g is not None else None
        return LayerCache(g, kv, self.state.get(cache_id), self.page_size, write)

    def clear_pages(self, kernels, pages_per_group):
        """Pages that have just been handed out start at zero in every cache of their group: whatever the
        last holder left (which may not even be finite) must not meet a masked key's zero weight."""
        for g, pages in enumerate(pages_per_group):
            if pages:
                kernels.clear_pages(self.kv[g], pages)

    def clear_state(self, slot: int):
        """A new request takes `slot`: its fixed-size state starts at zero."""
        for t in self.state.values():
            t[slot].zero_()
