"""Paged key/value cache manager: pools of pages, block tables, per-request state slots.

The reference keeps one contiguous key and one value buffer per layer per *slot*
(src/gpu_model.rs:745-746) and frees nothing until the slot is reused.  This manager is
the paged design instead:

* a **cache group** is a set of mixer calls with the same per-token need (all keys, or
  a window of them); each group has its own pool of fixed-size pages and, per request,
  a **block table** mapping logical page number (position // page_size) to a physical
  page, -1 where no page is held;
* pages are taken before a step writes into them (:meth:`CacheManager.reserve`), and
  given back when the request ends (:meth:`release`) or, in a window group, once every
  position of the page is older than the window (:meth:`commit`);
* free pages are handed out most-recently-freed first, so reuse happens quickly and
  tests can force it;
* every request also holds one **state slot**, an index into per-call arrays of
  fixed-size state, from admission to release.

The manager is host-side bookkeeping only and has no knowledge of tensors; the engine
owns the device storage the page numbers index.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence


class OutOfPages(RuntimeError):
    """A group's pool cannot supply the pages a step needs."""


class OutOfSlots(RuntimeError):
    """All state slots are taken."""


class PagePool:
    """Free list of page numbers 0..n-1, most recently freed first."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() hands out 0 first
        self._held = [False] * num_pages
        self.allocations = 0           # pages handed out so far
        self.reuses = 0                # of which had been used before
        self._ever_used = [False] * num_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.pop()
        assert not self._held[p], f"page {p} handed out twice"
        self._held[p] = True
        self.allocations += 1
        if self._ever_used[p]:
            self.reuses += 1
        self._ever_used[p] = True
        return p

    def give_back(self, p: int) -> None:
        if not 0 <= p < self.num_pages or not self._held[p]:
            raise RuntimeError(f"page {p} given back but not held")
        self._held[p] = False
        self._free.append(p)

    def held_pages(self) -> List[int]:
        return [i for i, h in enumerate(self._held) if h]


@dataclass
class GroupNeed:
    """What a cache group needs to know to place tokens: the window, or None for all keys."""
    window: Optional[int] = None


@dataclass
class _Request:
    slot: int
    length: int = 0                                   # tokens committed
    reserved: int = 0                                 # tokens that have pages (>= length)
    tables: List[List[int]] = field(default_factory=list)   # per group: logical page → physical or -1


class CacheManager:
    def __init__(self, groups: Sequence[GroupNeed], page_size: int, num_pages: int, max_seqs: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups = list(groups)
        self.pools = [PagePool(num_pages) for _ in self.groups]
        self.max_seqs = max_seqs
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}

    # ------------------------------------------------------------ admission / release
    def admit(self, rid: Hashable) -> int:
        """Registers a request and gives it a state slot (the caller zeroes the slot's state)."""
        if rid in self._requests:
            raise KeyError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_seqs} state slots are taken")
        slot = self._free_slots.pop()
        self._requests[rid] = _Request(slot=slot, tables=[[] for _ in self.groups])
        return slot

    def release(self, rid: Hashable) -> None:
        """Gives back every page and the state slot of a request."""
        r = self._requests.pop(rid)
        for pool, table in zip(self.pools, r.tables):
            for p in table:
                if p >= 0:
                    pool.give_back(p)
        self._free_slots.append(r.slot)

    def is_live(self, rid: Hashable) -> bool:
        return rid in self._requests

    def live(self) -> List[Hashable]:
        return list(self._requests)

    # ------------------------------------------------------------ queries
    def length(self, rid: Hashable) -> int:
        return self._requests[rid].length

    def slot(self, rid: Hashable) -> int:
        return self._requests[rid].slot

    def table(self, rid: Hashable, group: int) -> List[int]:
        return self._requests[rid].tables[group]

    def n_free(self, group: int) -> int:
        return self.pools[group].n_free

    def _first_needed_page(self, group: int, first_query_pos: int) -> int:
        """Lowest logical page a query at ``first_query_pos`` can still read in this group."""
        w = self.groups[group].window
        if w is None:
            return 0
        return max(0, first_query_pos - w + 1) // self.page_size

    def pages_to_reserve(self, rid: Hashable, n_new: int) -> List[int]:
        """Per group, the pages :meth:`reserve` would take for ``n_new`` more tokens."""
        r = self._requests[rid]
        end = max(r.reserved, r.length + n_new)
        need = []
        for g, table in enumerate(r.tables):
            last = (end - 1) // self.page_size if end > 0 else -1
            need.append(max(0, last + 1 - len(table)))
        return need

    def can_reserve(self, rid: Hashable, n_new: int, spare: Optional[List[int]] = None) -> bool:
        """Whether the pools (minus ``spare`` pages per group already promised elsewhere) can supply them."""
        need = self.pages_to_reserve(rid, n_new)
        return all(n <= self.pools[g].n_free - (spare[g] if spare else 0) for g, n in enumerate(need))

    # ------------------------------------------------------------ step protocol
    def reserve(self, rid: Hashable, n_new: int) -> None:
        """Takes the pages positions [length, length + n_new) need in every group, all or nothing."""
        r = self._requests[rid]
        if n_new <= 0:
            raise ValueError("reserve needs at least one token")
        need = self.pages_to_reserve(rid, n_new)
        for g, n in enumerate(need):
            if n > self.pools[g].n_free:
                raise OutOfPages(f"request {rid!r} needs {n} more pages in cache group {g}, "
                                 f"{self.pools[g].n_free} are free")
        for g, n in enumerate(need):
            for _ in range(n):
                r.tables[g].append(self.pools[g].take())
        r.reserved = max(r.reserved, r.length + n_new)

    def commit(self, rid: Hashable, n_new: int) -> None:
        """The step wrote ``n_new`` tokens: advances the length and gives back pages a window has passed."""
        r = self._requests[rid]
        if r.length + n_new > r.reserved:
            raise RuntimeError(f"request {rid!r}: committing {n_new} tokens beyond the reserved {r.reserved}")
        r.length += n_new
        for g, table in enumerate(r.tables):
            first = min(self._first_needed_page(g, r.length), len(table))   # the next query sits at r.length
            for lp in range(first):
                if table[lp] >= 0:
                    self.pools[g].give_back(table[lp])
                    table[lp] = -1

    def rollback(self, rid: Hashable) -> None:
        """Gives back pages reserved beyond the committed length (a step that did not run)."""
        r = self._requests[rid]
        keep = (r.length + self.page_size - 1) // self.page_size
        for g, table in enumerate(r.tables):
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    self.pools[g].give_back(p)
        r.reserved = r.length

    # ------------------------------------------------------------ invariants (used by tests)
    def check(self) -> None:
        """No page lost, none held twice: held pages of each pool = pages in live tables, each once."""
        for g, pool in enumerate(self.pools):
            seen = []
            for r in self._requests.values():
                seen += [p for p in r.tables[g] if p >= 0]
            assert len(seen) == len(set(seen)), f"group {g}: a page is in two tables"
            assert sorted(seen) == pool.held_pages(), f"group {g}: tables and pool disagree"
            assert len(seen) + pool.n_free == pool.num_pages, f"group {g}: pages lost"
        slots = [r.slot for r in self._requests.values()]
        assert len(slots) == len(set(slots)), "a state slot is held twice"
        assert len(slots) + len(self._free_slots) == self.max_seqs, "state slots lost"
