"""Cache manager: pages of keys and values for groups of layers, and slots of per-request state.

Layers whose caches have the same needs (kv heads, head size, all keys or a window of W keys)
form a group.  A group has its own pool of pages and, for every request, its own block table;
one page id is valid in every layer of its group.  Pages go back to the pool when a request
ends, when it is preempted, and, in a window group, as soon as the window has passed them.
Beside the pages every request holds one slot of fixed-size state for mixers that ask for it.

lucciola has one group (every layer keeps all keys), takes pages when a request crosses a page
boundary or for a whole portion of a prompt at once (src/scheduler.cc:55-58, 89-97) and gives
them back when the request ends or is preempted (src/scheduler.cc:20-40); the same rules hold
here for each group.  Everything in this file is host bookkeeping; device memory is in
device_cache.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Hashable, Sequence

from ..parts.base import KVPages, StateSlot
from .page_pool import PagePool, PagePoolError

NO_PAGE = -1


@dataclass(frozen=True)
class CacheGroup:
    num_kv_heads: int
    head_dim: int
    window: int                      # 0: all keys
    cache_ids: tuple[int, ...]       # the model's cache ids that live in this group


def plan_groups(requests: Sequence[KVPages | StateSlot | None]) -> tuple[list[CacheGroup], list[int]]:
    """Group the model's caches by their needs.  Returns the groups and the cache ids that hold state."""
    by_key: dict[tuple[int, int, int], list[int]] = {}
    state_ids: list[int] = []
    for cid, r in enumerate(requests):
        if isinstance(r, KVPages):
            by_key.setdefault((r.num_kv_heads, r.head_dim, r.window), []).append(cid)
        elif isinstance(r, StateSlot):
            state_ids.append(cid)
    groups = [CacheGroup(k[0], k[1], k[2], tuple(v)) for k, v in by_key.items()]
    return groups, state_ids


@dataclass
class _RequestCache:
    slot: int
    tables: list[list[int]]          # per group: page of each logical page index, NO_PAGE once released
    length: int = 0                  # tokens whose keys are (or are about to be) in the cache
    version: int = 0                 # new, manager-wide unique number whenever a table changes (lets callers cache a converted copy)


class CacheManager:
    def __init__(self, groups: Sequence[CacheGroup], page_size: int, num_pages: int | Sequence[int], num_slots: int):
        self.groups = list(groups)
        self.page_size = page_size
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        self.pools = [PagePool(n) for n in counts]
        self.num_slots = num_slots
        self._free_slots = list(range(num_slots - 1, -1, -1))
        self._requests: dict[Hashable, _RequestCache] = {}
        self._versions = 0

    # ---- requests ------------------------------------------------------
    def has_request(self, rid: Hashable) -> bool:
        return rid in self._requests

    def can_admit(self) -> bool:
        return bool(self._free_slots)

    def admit(self, rid: Hashable) -> int:
        """Give a new request its state slot and empty block tables."""
        if rid in self._requests:
            raise PagePoolError(f"request {rid!r} is already admitted")
        if not self._free_slots:
            raise PagePoolError("no free state slot")
        slot = self._free_slots.pop()
        self._versions += 1
        self._requests[rid] = _RequestCache(slot, [[] for _ in self.groups], version=self._versions)
        return slot

    def release(self, rid: Hashable) -> None:
        """Give back everything a request holds (it ended or is preempted)."""
        rc = self._requests.pop(rid)
        for g, table in enumerate(rc.tables):
            for p in table:
                if p != NO_PAGE:
                    self.pools[g].free(p)
        self._free_slots.append(rc.slot)

    # ---- pages ---------------------------------------------------------
    def _first_needed_page(self, g: int, start: int) -> int:
        """Index of the first page a query at position `start` can still see in group g."""
        w = self.groups[g].window
        return max(0, start - w + 1) // self.page_size if w > 0 else 0

    def pages_needed(self, rid: Hashable, new_length: int) -> list[int]:
        """Pages each group has to take so that positions below new_length are backed."""
        rc = self._requests[rid]
        want = -(-new_length // self.page_size)
        return [max(0, want - len(t)) for t in rc.tables]

    def can_extend(self, rid: Hashable, new_length: int) -> bool:
        return all(self.pools[g].can_allocate(n) for g, n in enumerate(self.pages_needed(rid, new_length)))

    def extend(self, rid: Hashable, new_length: int) -> bool:
        """Take the pages for positions [length, new_length) in every group, all or nothing."""
        rc = self._requests[rid]
        if new_length < rc.length:
            raise PagePoolError(f"request {rid!r} cannot shrink from {rc.length} to {new_length}")
        need = self.pages_needed(rid, new_length)
        if not all(self.pools[g].can_allocate(n) for g, n in enumerate(need)):
            return False
        for g, n in enumerate(need):
            for _ in range(n):
                rc.tables[g].append(self.pools[g].allocate())
        if any(need):
            self._versions += 1
            rc.version = self._versions
        rc.length = new_length
        return True

    def extend_by_one(self, rids: Sequence[Hashable]) -> Optional[list[int]]:
        """One more position for each of these admitted requests, all or nothing: the step of a decoding batch.
        Returns the positions the new tokens take (the lengths before), or None when a group lacks the pages."""
        ps = self.page_size
        reqs = [self._requests[rid] for rid in rids]
        need = [0] * len(self.groups)
        for rc in reqs:
            want = rc.length // ps + 1                       # pages that back positions 0 .. length
            for g, t in enumerate(rc.tables):
                if want > len(t):
                    need[g] += want - len(t)
        if any(need) and not all(self.pools[g].can_allocate(n) for g, n in enumerate(need)):
            return None
        starts = []
        for rc in reqs:
            want = rc.length // ps + 1
            grew = False
            for g, t in enumerate(rc.tables):
                while len(t) < want:
                    t.append(self.pools[g].allocate())
                    grew = True
            if grew:
                self._versions += 1
                rc.version = self._versions
            starts.append(rc.length)
            rc.length += 1
        return starts

    def retract_by_one(self, rids: Sequence[Hashable]) -> None:
        """Undo extend_by_one for a step that was prepared and will not run.  A page that was taken for the position
        stays in the request's table (the position's next step finds it there; a request that ends gives it back)."""
        for rid in rids:
            rc = self._requests.get(rid)
            if rc is not None and rc.length > 0:
                rc.length -= 1

    def max_extension(self, rid: Hashable, upto: int) -> int:
        """The largest length <= upto that the free pages allow for this request."""
        rc = self._requests[rid]
        best = upto
        for g, t in enumerate(rc.tables):
            best = min(best, (len(t) + self.pools[g].num_free) * self.page_size)
        return max(min(best, upto), rc.length)

    def release_behind_window(self, rid: Hashable) -> int:
        """After a step: free the pages that no later query of this request can see.  Returns how many."""
        rc = self._requests[rid]
        freed = 0
        for g, table in enumerate(rc.tables):
            if self.groups[g].window <= 0:
                continue
            first = min(self._first_needed_page(g, rc.length), len(table))
            for i in range(first):
                if table[i] != NO_PAGE:
                    self.pools[g].free(table[i])
                    table[i] = NO_PAGE
                    freed += 1
        if freed:
            self._versions += 1
            rc.version = self._versions
        return freed

    # ---- views ---------------------------------------------------------
    def length(self, rid: Hashable) -> int:
        return self._requests[rid].length

    def slot(self, rid: Hashable) -> int:
        return self._requests[rid].slot

    def block_table(self, rid: Hashable, group: int) -> list[int]:
        return self._requests[rid].tables[group]

    def version(self, rid: Hashable) -> int:
        return self._requests[rid].version

    def num_requests(self) -> int:
        return len(self._requests)

    def check_invariants(self) -> None:
        """No page lost, none held twice: every page is free or in exactly one table."""
        for g, pool in enumerate(self.pools):
            seen: set[int] = set()
            for rid, rc in self._requests.items():
                for p in rc.tables[g]:
                    if p == NO_PAGE:
                        continue
                    if p in seen:
                        raise PagePoolError(f"page {p} of group {g} is held twice")
                    seen.add(p)
            free = set(pool._free)
            if len(free) != len(pool._free):
                raise PagePoolError(f"group {g}: a page is twice in the free list")
            if seen & free:
                raise PagePoolError(f"group {g}: pages {sorted(seen & free)} are both held and free")
            if len(seen) + len(free) != pool.num_pages:
                raise PagePoolError(f"group {g}: {pool.num_pages - len(seen) - len(free)} page(s) lost")
        slots = [rc.slot for rc in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PagePoolError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.num_slots:
            raise PagePoolError("a state slot is lost")
