"""Cache manager: pages of keys and values per cache group, block tables per request, state slots.

What 7QiC/ccInfer's manager does is kept where it applies: pages of a fixed
number of tokens, a FIFO free list (src/cache/kv_cache_manager.cpp:78-82,
242-244), pages taken on demand just before a step
(src/worker/batch_translator.cpp:196-211), everything of a request given back
when it ends (src/worker/worker.cpp:317-326), validate-then-mutate on release
with double-free detection (src/cache/kv_cache_manager.cpp:216-230), and a
transactional step: pages taken for a step that fails are returned
(src/worker/batch_translator.cpp:72-75, 579-589).  Prefix sharing, reference
counts and the LRU list are left out: a page has exactly one owner.

Beyond the reference:

* cache groups.  Layers whose mixers need the same thing (all keys, or a
  window of W keys) form a group with a page pool and block tables of its own.
  In a window group the pages that every later query has passed are given
  back while the request still runs.
* state slots.  A request gets a slot id when it is opened; the slot indexes
  per-request state tensors of fixed size (for mixers that have such state)
  and is returned when the request is closed.

Everything here is host-side bookkeeping; the device tensors (one set per
layer that keeps a cache) belong to the engine.
"""
from __future__ import annotations

import collections
import dataclasses
from typing import Dict, Hashable, List, Optional, Tuple

import numpy as np

from ..errors import (InvalidArgument, KVBlockDoubleFree, KVBlockExhausted, KVInvalidBlockTable, SlotExhausted)


@dataclasses.dataclass(frozen=True)
class GroupSpec:
    """A cache group: which keys its layers read (``window`` None = all) and its pool."""
    key: Tuple
    window: Optional[int]
    page_size: int
    num_pages: int


class PagePool:
    """Pages of one group: FIFO free list and an owner per page."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise InvalidArgument("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = collections.deque(range(num_pages))
        self._owner: List[Optional[Hashable]] = [None] * num_pages
        self.high_water = 0

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, owner: Hashable, n: int) -> List[int]:
        if n < 0:
            raise InvalidArgument("cannot take a negative number of pages")
        if n > len(self._free):
            raise KVBlockExhausted(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.popleft() for _ in range(n)]
        for p in pages:
            self._owner[p] = owner
        self.high_water = max(self.high_water, self.used_pages)
        return pages

    def give_back(self, owner: Hashable, pages: List[int]) -> None:
        """All-or-nothing: checks every page before any is freed."""
        seen = set()
        for p in pages:
            if not isinstance(p, int) or not (0 <= p < self.num_pages):
                raise KVInvalidBlockTable(f"page id {p!r} is outside the pool of {self.num_pages}")
            if p in seen:
                raise KVBlockDoubleFree(f"page {p} is named twice in one release")
            if self._owner[p] is None:
                raise KVBlockDoubleFree(f"page {p} is already free")
            if self._owner[p] != owner:
                raise KVInvalidBlockTable(f"page {p} belongs to {self._owner[p]!r}, not to {owner!r}")
            seen.add(p)
        for p in pages:
            self._owner[p] = None
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner[page]


class SlotPool:
    """Fixed number of per-request state slots."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise InvalidArgument("at least one state slot is needed")
        self.num_slots = num_slots
        self._free = collections.deque(range(num_slots))
        self._used = [False] * num_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise SlotExhausted(f"all {self.num_slots} request slots are in use")
        s = self._free.popleft()
        self._used[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots):
            raise InvalidArgument(f"slot {slot} is outside the pool of {self.num_slots}")
        if not self._used[slot]:
            raise KVBlockDoubleFree(f"slot {slot} is already free")
        self._used[slot] = False
        self._free.append(slot)


class RequestCache:
    """What one request holds: its slot, how many tokens are cached, and per group a block table.

    ``tables[g][i]`` is the physical page of logical page i (tokens i*P .. i*P+P-1) or -1
    when that page was never needed or has been given back (window groups)."""

    def __init__(self, req_id: Hashable, slot: int, n_groups: int):
        self.req_id = req_id
        self.slot = slot
        self.ctx_len = 0
        self.tables: List[List[int]] = [[] for _ in range(n_groups)]
        # the same tables as int32 arrays (with spare capacity), kept in step by the manager: what the step
        # function copies into its pinned buffer without walking a Python list per request and step
        self._arrays: List[np.ndarray] = [np.full(16, -1, dtype=np.int32) for _ in range(n_groups)]
        # pages taken by reserve() and not yet committed: [(group, logical index)]
        self._pending: List[Tuple[int, int]] = []
        self._pending_tokens = 0

    def pages_held(self, g: int) -> int:
        return sum(1 for p in self.tables[g] if p >= 0)

    def table_array(self, g: int) -> np.ndarray:
        """The block table of group g as an int32 array (a view: do not keep it across steps)."""
        return self._arrays[g][:len(self.tables[g])]

    def _append(self, g: int, page: int) -> None:
        n = len(self.tables[g])
        if n == self._arrays[g].size:
            grown = np.full(2 * n, -1, dtype=np.int32)
            grown[:n] = self._arrays[g]
            self._arrays[g] = grown
        self._arrays[g][n] = page
        self.tables[g].append(page)

    def _pop(self, g: int) -> None:
        self.tables[g].pop()

    def _drop(self, g: int, i: int) -> None:
        self.tables[g][i] = -1
        self._arrays[g][i] = -1


class CacheManager:
    def __init__(self, groups: List[GroupSpec], max_requests: int):
        self.groups = list(groups)
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        self.slots = SlotPool(max_requests)
        self.requests: Dict[Hashable, RequestCache] = {}

    # -- requests ----------------------------------------------------------------
    def open(self, req_id: Hashable) -> RequestCache:
        if req_id in self.requests:
            raise InvalidArgument(f"request {req_id!r} is already open")
        rc = RequestCache(req_id, self.slots.take(), len(self.groups))
        self.requests[req_id] = rc
        return rc

    def get(self, req_id: Hashable) -> RequestCache:
        try:
            return self.requests[req_id]
        except KeyError:
            raise InvalidArgument(f"request {req_id!r} is not open") from None

    def close(self, req_id: Hashable) -> None:
        """Gives back every page and the slot of a request."""
        rc = self.get(req_id)
        for g, pool in enumerate(self.pools):
            pool.give_back(req_id, [p for p in rc.tables[g] if p >= 0])
            rc.tables[g] = []
            rc._arrays[g] = np.full(16, -1, dtype=np.int32)
        self.slots.give_back(rc.slot)
        del self.requests[req_id]

    # -- page arithmetic -----------------------------------------------------------
    def first_needed_page(self, g: int, ctx_len: int) -> int:
        """Logical index of the first page a query at position >= ctx_len can still read."""
        spec = self.groups[g]
        if spec.window is None:
            return 0
        first_key = ctx_len - spec.window + 1
        return max(0, first_key) // spec.page_size

    def pages_needed(self, req_id: Hashable, n_new: int) -> List[int]:
        """Pages each group would have to take to hold ``n_new`` more tokens of the request."""
        rc = self.get(req_id)
        return [self._pages_needed(rc, g, n_new) for g in range(len(self.groups))]

    def pages_needed_for(self, ctx_len: int, n_new: int, g: int) -> int:
        """Same for a request described by its length only (nothing held beyond ctx_len's pages)."""
        P = self.groups[g].page_size
        have = -(-ctx_len // P)
        return -(-(ctx_len + n_new) // P) - have

    def _pages_needed(self, rc: RequestCache, g: int, n_new: int) -> int:
        P = self.groups[g].page_size
        return max(0, -(-(rc.ctx_len + n_new) // P) - len(rc.tables[g]))

    # -- a step: reserve, then commit or roll back ------------------------------------
    def reserve(self, req_id: Hashable, n_new: int) -> None:
        """Takes the pages for tokens ctx_len .. ctx_len + n_new - 1 in every group.

        Either all groups get their pages or none keeps any (KVBlockExhausted)."""
        rc = self.get(req_id)
        if n_new <= 0:
            raise InvalidArgument("a step brings at least one token per request")
        if rc._pending_tokens:
            raise InvalidArgument(f"request {req_id!r} has an uncommitted reservation")
        taken: List[Tuple[int, int]] = []
        try:
            for g, pool in enumerate(self.pools):
                n = self._pages_needed(rc, g, n_new)
                pages = pool.take(req_id, n)
                for p in pages:
                    rc._append(g, p)
                    taken.append((g, len(rc.tables[g]) - 1))
        except KVBlockExhausted:
            self._undo(rc, taken)
            raise
        rc._pending = taken
        rc._pending_tokens = n_new

    def _undo(self, rc: RequestCache, taken: List[Tuple[int, int]]) -> None:
        for g in range(len(self.groups)):
            idx = sorted((i for gg, i in taken if gg == g), reverse=True)
            pages = [rc.tables[g][i] for i in idx]
            self.pools[g].give_back(rc.req_id, pages)
            for i in idx:  # they are the tail of the table
                assert i == len(rc.tables[g]) - 1
                rc._pop(g)

    def rollback(self, req_id: Hashable) -> None:
        """Returns the pages of a reservation whose step did not happen."""
        rc = self.get(req_id)
        self._undo(rc, rc._pending)
        rc._pending, rc._pending_tokens = [], 0

    def commit(self, req_id: Hashable) -> None:
        """The step ran: the tokens are cached; window groups give back pages every later query has passed."""
        rc = self.get(req_id)
        if not rc._pending_tokens:
            raise InvalidArgument(f"request {req_id!r} has nothing reserved")
        rc.ctx_len += rc._pending_tokens
        rc._pending, rc._pending_tokens = [], 0
        for g, spec in enumerate(self.groups):
            if spec.window is None:
                continue
            first = min(self.first_needed_page(g, rc.ctx_len), len(rc.tables[g]))
            stale = [i for i in range(first) if rc.tables[g][i] >= 0]
            if stale:
                self.pools[g].give_back(req_id, [rc.tables[g][i] for i in stale])
                for i in stale:
                    rc._drop(g, i)

    # -- addressing -------------------------------------------------------------------
    def slot_of(self, rc: RequestCache, g: int, position: int) -> int:
        """Cache slot (page * page_size + offset) of a token position, which must be held."""
        P = self.groups[g].page_size
        page = rc.tables[g][position // P]
        if page < 0:
            raise KVInvalidBlockTable(f"position {position} of request {rc.req_id!r} is no longer cached")
        return page * P + position % P

    # -- figures ------------------------------------------------------------------------
    def stats(self) -> dict:
        return {
            "requests": len(self.requests),
            "slots_total": self.slots.num_slots,
            "slots_free": self.slots.free_slots,
            "groups": [
                {"key": list(map(str, g.key)), "window": g.window, "page_size": g.page_size,
                 "pages_total": pool.num_pages, "pages_free": pool.free_pages, "pages_used": pool.used_pages,
                 "pages_high_water": pool.high_water}
                for g, pool in zip(self.groups, self.pools)],
        }

    def check_consistency(self) -> None:
        """Every page is free or in exactly one table of its owner (used by tests)."""
        for g, pool in enumerate(self.pools):
            held = {}
            for rc in self.requests.values():
                for p in rc.tables[g]:
                    if p >= 0:
                        if p in held:
                            raise AssertionError(f"group {g}: page {p} held by {held[p]!r} and {rc.req_id!r}")
                        held[p] = rc.req_id
            free = list(pool._free)
            if len(set(free)) != len(free):
                raise AssertionError(f"group {g}: a page is on the free list twice")
            if set(free) & set(held):
                raise AssertionError(f"group {g}: pages both free and held: {set(free) & set(held)}")
            if len(free) + len(held) != pool.num_pages:
                raise AssertionError(f"group {g}: {pool.num_pages - len(free) - len(held)} pages lost")
            for p, owner in held.items():
                if pool.owner_of(p) != owner:
                    raise AssertionError(f"group {g}: page {p} owner mismatch")
            for rc in self.requests.values():
                if rc.table_array(g).tolist() != rc.tables[g]:
                    raise AssertionError(f"group {g}: the array of request {rc.req_id!r} differs from its table")
