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
from .manager import CacheGroup


def bytes_per_page(groups: Sequence[CacheGroup], page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id costs when every group gets the same number of pages."""
    el = torch.empty((), dtype=dtype).element_size()
    return sum(len(g.cache_ids) * 2 * g.num_kv_heads * page_size * g.head_dim * el for g in groups)


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
        self.views: list[object] = [None] * len(requests)
        for gi, g in enumerate(groups):
            pool = torch.zeros((len(g.cache_ids), 2, num_pages[gi], g.num_kv_heads, page_size, g.head_dim),
                               dtype=dtype, device=device)
            self.pools.append(pool)
            for li, cid in enumerate(g.cache_ids):
                self.views[cid] = KVCacheView(pool[li, 0], pool[li, 1], gi, page_size)
        self.states: dict[int, torch.Tensor] = {}
        for cid, r in enumerate(requests):
            if isinstance(r, StateSlot):
                # one row more than there are slots: row `num_slots` belongs to no request; the entries that pad a
                # recorded step read and write it
                st = torch.zeros((num_slots + 1, *r.shape), dtype=r.dtype, device=device)
                self.states[cid] = st
                self.views[cid] = StateCacheView(st)

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
