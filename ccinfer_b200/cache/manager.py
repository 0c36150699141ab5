"""Cache manager: pages per cache group, block tables per request, state slots.

The bookkeeping itself is native: ``csrc/host/host_core.cpp`` behind the C interface of
``csrc/host/ccinfer.h``; the classes here give it the package's names and exceptions and let requests be
named by any hashable id.  What 7QiC/ccInfer's manager does is kept where it applies: pages of a fixed number
of tokens, a FIFO free list (src/cache/kv_cache_manager.cpp:78-82, 242-244), pages taken on demand just
before a step (src/worker/batch_translator.cpp:196-211), everything of a request given back when it ends
(src/worker/worker.cpp:317-326), validate-then-mutate on release with double-free detection
(src/cache/kv_cache_manager.cpp:216-230), and a transactional step: pages taken for a step that fails are
returned (src/worker/batch_translator.cpp:72-75, 579-589).  Prefix sharing, reference counts and the LRU list
are left out: a page has exactly one owner.

Beyond the reference:

* cache groups.  Layers whose mixers need the same thing (all tokens, or a window of W) form a group with a
  page pool and block tables of its own.  In a window group the pages that every later query has passed are
  given back while the request still runs.
* state slots.  A request gets a slot id when it is opened; the slot indexes per-request state tensors of
  fixed size (for mixers that have such state) and is returned when the request is closed.

Everything here is host-side bookkeeping; the device tensors (one set per layer that keeps a cache) belong to
the engine.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Hashable, List, Optional, Tuple

import numpy as np

from ..errors import InvalidArgument, KVInvalidBlockTable
from ..native import HostCore


@dataclasses.dataclass(frozen=True)
class GroupSpec:
    """A cache group: which tokens its layers read (``window`` None = all) and its pool."""
    key: Tuple
    window: Optional[int]
    page_size: int
    num_pages: int


class _Names:
    """Hashable ids <-> the 64-bit numbers by which the host core knows owners and sequences."""

    def __init__(self):
        self._num: Dict[Hashable, int] = {}
        self._next = 1

    def number(self, name: Hashable, create: bool = True) -> int:
        n = self._num.get(name)
        if n is None:
            if not create:
                return 0   # a number nobody has
            n = self._num[name] = self._next
            self._next += 1
        return n

    def forget(self, name: Hashable) -> None:
        self._num.pop(name, None)


class PagePool:
    """Pages of one group: FIFO free list and an owner per page."""

    def __init__(self, num_pages: int, _core: HostCore = None, _group: int = 0, _names: _Names = None):
        self._core = _core or HostCore([(None, 1, num_pages)], 1, 1, max(1, num_pages))
        self._g = _group
        self._names = _names or _Names()
        self.num_pages = self._core.stats().pages_total[self._g]

    @property
    def free_pages(self) -> int:
        return self._core.stats().pages_free[self._g]

    @property
    def used_pages(self) -> int:
        return self.num_pages - self.free_pages

    @property
    def high_water(self) -> int:
        return self._core.stats().pages_high_water[self._g]

    def take(self, owner: Hashable, n: int) -> List[int]:
        return self._core.pool_take(self._g, self._names.number(owner), n)

    def give_back(self, owner: Hashable, pages: List[int]) -> None:
        """All-or-nothing: every page is checked before any is freed."""
        self._core.pool_give_back(self._g, self._names.number(owner), list(pages))

    def owner_of(self, page: int):
        n = self._core.pool_owner(self._g, page)
        if n is None:
            return None
        for name, num in self._names._num.items():
            if num == n:
                return name
        return n


class SlotPool:
    """Fixed number of per-request state slots."""

    def __init__(self, num_slots: int, _core: HostCore = None):
        self._core = _core or HostCore([], num_slots, max(1, num_slots), 1)
        self.num_slots = self._core.stats().slots_total

    @property
    def free_slots(self) -> int:
        return self._core.stats().slots_free

    def take(self) -> int:
        return self._core.slot_take()

    def give_back(self, slot: int) -> None:
        self._core.slot_give_back(int(slot))


class RequestCache:
    """What one request holds: its slot, how many tokens are cached, and per group a block table.

    ``tables[g][i]`` is the physical page of logical page i (tokens i*P .. i*P+P-1) or -1 when that page has
    been given back (window groups)."""

    def __init__(self, core: HostCore, req_id: Hashable, seq: int, slot: int, n_groups: int):
        self._core, self.req_id, self.seq, self.slot, self._n_groups = core, req_id, seq, slot, n_groups

    @property
    def ctx_len(self) -> int:
        return self._core.seq_state(self.seq)[1]

    @property
    def tables(self) -> List[List[int]]:
        return [self._core.block_table(self.seq, g) for g in range(self._n_groups)]

    def table_len(self, g: int) -> int:
        """Logical pages the table of group g spans (given-back ones included)."""
        return self._core.table_len(self.seq, g)

    def table_array(self, g: int) -> np.ndarray:
        return np.asarray(self._core.block_table(self.seq, g), dtype=np.int32)

    def pages_held(self, g: int) -> int:
        return sum(1 for p in self._core.block_table(self.seq, g) if p >= 0)


class CacheManager:
    def __init__(self, groups: List[GroupSpec], max_requests: int, max_tokens_per_step: int = None,
                 max_context: int = None):
        """``max_tokens_per_step`` and ``max_context`` size the step arrays that the host core lays out (the
        engine names them; the defaults serve a manager used for its bookkeeping alone)."""
        self.groups = list(groups)
        if max_requests <= 0:
            raise InvalidArgument("at least one state slot is needed")
        if max_context is None:
            max_context = max([g.num_pages * g.page_size for g in self.groups if g.window is None] or
                              [g.num_pages * g.page_size for g in self.groups] or [1])
        self.core = HostCore([(g.window, g.page_size, g.num_pages) for g in self.groups], max_requests,
                             max_tokens_per_step or max(max_requests, 1), max(1, max_context))
        self._names = _Names()
        self.pools = [PagePool(g.num_pages, self.core, i, self._names) for i, g in enumerate(self.groups)]
        self.slots = SlotPool(max_requests, self.core)
        self.requests: Dict[Hashable, RequestCache] = {}

    # -- requests ----------------------------------------------------------------
    def open(self, req_id: Hashable) -> RequestCache:
        if req_id in self.requests:
            raise InvalidArgument(f"request {req_id!r} is already open")
        seq = self._names.number(req_id)
        rc = RequestCache(self.core, req_id, seq, self.core.alloc_seq(seq), len(self.groups))
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
        self.core.free_seq(rc.seq)
        del self.requests[req_id]
        self._names.forget(req_id)

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
        return self.core.pages_needed(self.get(req_id).seq, n_new)

    def pages_needed_for(self, ctx_len: int, n_new: int, g: int) -> int:
        """Same for a request described by its length only (nothing held beyond ctx_len's pages)."""
        P = self.groups[g].page_size
        have = -(-ctx_len // P)
        return -(-(ctx_len + n_new) // P) - have

    # -- a step: reserve, then commit or roll back ------------------------------------
    def reserve(self, req_id: Hashable, n_new: int) -> None:
        """Takes the pages for tokens ctx_len .. ctx_len + n_new - 1 in every group.

        Either all groups get their pages or none keeps any (KVBlockExhausted)."""
        self.core.reserve(self.get(req_id).seq, n_new)

    def rollback(self, req_id: Hashable) -> None:
        """Returns the pages of a reservation whose step did not happen."""
        self.core.rollback(self.get(req_id).seq)

    def commit(self, req_id: Hashable) -> None:
        """The step ran: the tokens are cached; window groups give back pages every later query has passed."""
        self.core.commit(self.get(req_id).seq)

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
        st = self.core.stats()
        return {
            "requests": st.seqs,
            "slots_total": st.slots_total,
            "slots_free": st.slots_free,
            "groups": [
                {"key": list(map(str, g.key)), "window": g.window, "page_size": g.page_size,
                 "pages_total": st.pages_total[i], "pages_free": st.pages_free[i],
                 "pages_used": st.pages_total[i] - st.pages_free[i], "pages_high_water": st.pages_high_water[i]}
                for i, g in enumerate(self.groups)],
        }

    def check_consistency(self) -> None:
        """Every page is free or in exactly one table of its owner, none is lost (used by tests)."""
        self.core.check()
        for rid, rc in self.requests.items():
            if self.core.seq_state(rc.seq)[0] != rc.slot:
                raise AssertionError(f"request {rid!r}: its slot moved")
