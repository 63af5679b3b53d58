"""Device memory of the caches: one tensor of pages per group, one tensor of slots (and a spare row) per state cache.

Pages of a group: [layer in group][k|v][page][kv head][slot in page][head_dim], so that the keys
(or values) of one page and kv head are one contiguous box of page_size x head_dim elements.
lucciola keeps [page][slot][kv head][head_dim] per layer (src/kernels/attention_paged.cu:33-36)
and sizes the pool as (free memory - 500 MB) * 0.9 / bytes of a page over all layers
(src/qwen.cc:527-557); `pages_that_fit` does the same count.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..parts.base import KVCacheView, KVPages, StateCacheView, StateSlot
from .manager import CacheGroup, flat_requests


def bytes_per_page(groups: Sequence[CacheGroup], page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id costs when every group gets the same number of pages."""
    el = torch.empty((), dtype=dtype).element_size()
    return sum(len(g.cache_ids) * g.num_kv_heads * page_size * (g.head_dim + (0 if g.shared else (g.v_head_dim or g.head_dim))) * el // max(1, g.every)
               for g in groups)


def pages_that_fit(groups: Sequence[CacheGroup], page_size: int, dtype: torch.dtype, device: torch.device,
                   fraction: float, reserve_bytes: int = 500 * 1024 * 1024) -> int:
    free, _ = torch.cuda.mem_get_info(device)
    per = bytes_per_page(groups, page_size, dtype)
    if per == 0:
        return 1
    return max(int((free - reserve_bytes) * fraction) // per, 0)


class DeviceCache:
    def __init__(self, requests: Sequence[KVPages | StateSlot | None], groups: Sequence[CacheGroup],
                 page_size: int, num_pages: Sequence[int], num_slots: int, dtype: torch.dtype, device: torch.device):
        self.page_size = page_size
        self.pools: list[torch.Tensor] = []
        single: dict[object, object] = {}
        self.value_pools: dict[int, torch.Tensor] = {}      # groups whose values have another size than their keys
        for gi, g in enumerate(groups):
            if g.v_head_dim and not g.shared:
                # keys and values in tensors of their own: [layer][page][kv head][slot][head_dim | v_head_dim]
                pool = torch.zeros((len(g.cache_ids), 1, num_pages[gi], g.num_kv_heads, page_size, g.head_dim), dtype=dtype, device=device)
                vpool = torch.zeros((len(g.cache_ids), num_pages[gi], g.num_kv_heads, page_size, g.v_head_dim), dtype=dtype, device=device)
                self.pools.append(pool)
                self.value_pools[gi] = vpool
                for li, key in enumerate(g.cache_ids):
                    single[key] = KVCacheView(pool[li, 0], vpool[li], gi, page_size)
                continue
            pool = torch.zeros((len(g.cache_ids), 1 if g.shared else 2, num_pages[gi], g.num_kv_heads, page_size, g.head_dim),
                               dtype=dtype, device=device)
            self.pools.append(pool)
            for li, key in enumerate(g.cache_ids):
                single[key] = KVCacheView(pool[li, 0], pool[li, 0 if g.shared else 1], gi, page_size)
        self.states: dict[object, torch.Tensor] = {}
        for key, r in flat_requests(requests):
            if isinstance(r, StateSlot):
                # one row more than there are slots: row `num_slots` belongs to no request; the entries that pad a
                # recorded step read and write it
                st = torch.zeros((num_slots + 1, *r.shape), dtype=r.dtype, device=device)
                self.states[key] = st
                single[key] = StateCacheView(st)
        # a cache id that asked for a tuple gets a tuple of views in the same order
        self.views: list[object] = [
            tuple(single.get((cid, j)) for j in range(len(r))) if isinstance(r, tuple) else single.get(cid)
            for cid, r in enumerate(requests)]

    def zero_slots(self, slots: torch.Tensor, stream: int) -> None:
        """Clear the state rows of newly admitted requests.  `slots`: int32 on the device, negative entries name
        no row (the list has a fixed length so that the launch can be part of a recorded step)."""
        from .. import ops
        for st in self.states.values():
            ops.zero_rows(st, slots, stream)

    def poison_pages(self, group: int, pages: Sequence[int], value: float = float("nan")) -> None:
        """Fill pages with a value that would show in any sum (for tests of page reuse)."""
        if pages:
            idx = torch.tensor(list(pages), dtype=torch.long, device=self.pools[group].device)
            self.pools[group][:, :, idx] = value
            if group in self.value_pools:
                self.value_pools[group][:, idx] = value

    def poison_slots(self, slots: Sequence[int], value: float = float("nan")) -> None:
        """Fill the state rows of these slots with a value that would show in any sum (for tests of slot reuse)."""
        for st in self.states.values():
            for slot in slots:
                st[slot] = value
