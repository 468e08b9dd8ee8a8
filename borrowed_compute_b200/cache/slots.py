"""Bookkeeping of the cache on the host: which sequence holds which slot and which pages.

A *slot* is one live sequence: its length and, for every storage group, the pages that
hold its positions (64 a page).  Pages come from a pool per group and go back to it when
the sequence ends, to be handed to the next one.  This module is plain Python and never
touches a device; the device side mirrors its page tables.

The reference keeps one growing buffer per conversation and drops the oldest of more than
16 (crates/bc-mesh/src/engine.rs:25,305-312; crates/bc-infer/src/gpu/mod.rs:404-423).
Here capacity is fixed when the engine is built, and running out is an error the caller
sees, never a silent eviction.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence

from ..config.errors import CacheError

PAGE = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


class PagePool:
    """Pages of one storage group: each is free or held, never both, never twice."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def available(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheError(f"the cache is full: {n} more pages of {PAGE} tokens are needed, {len(self._free)} are free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages or not self._held[p]:
                raise CacheError(f"page {p} is given back but is not held")
            self._held[p] = False
            self._free.append(p)

    def held(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


@dataclass
class GroupPlan:
    """What one storage group keeps per sequence: every position (window 0) or the last
    ``window`` of them."""

    window: int = 0


@dataclass
class _Slot:
    length: int = 0
    # per group: page index within the sequence -> page id, -1 where none is held
    pages: List[List[int]] = field(default_factory=list)


class SlotTable:
    """Slots and their pages across all storage groups.

    ``reserve(slot, n)`` makes room for the sequence to reach ``n`` positions and is what
    a step calls before its kernels write; ``commit`` records the new length afterwards.
    ``tables[g][slot]`` is the row a device page table mirrors; ``dirty`` names the
    (group, slot) rows changed since the mirror last looked.
    """

    def __init__(self, n_slots: int, n_pages: int, max_seq: int, groups: Sequence[GroupPlan]):
        if n_slots <= 0 or max_seq <= 0:
            raise CacheError(f"need at least one slot and one position, got {n_slots} slots, {max_seq} positions")
        self.n_slots, self.max_seq = n_slots, max_seq
        self.max_pages = pages_for(max_seq)
        self.groups = list(groups)
        self.pools = [PagePool(n_pages) for _ in self.groups]
        self._slots: Dict[int, _Slot] = {}
        self._free_slots: List[int] = list(range(n_slots - 1, -1, -1))
        self.tables: List[List[List[int]]] = [[[-1] * self.max_pages for _ in range(n_slots)] for _ in self.groups]
        self.dirty: set = set()

    # -- slots
    def acquire(self) -> int:
        if not self._free_slots:
            raise CacheError(f"all {self.n_slots} slots are in use")
        s = self._free_slots.pop()
        self._slots[s] = _Slot(0, [[] for _ in self.groups])
        return s

    def release(self, slot: int) -> None:
        st = self._held(slot)
        for g, pages in enumerate(st.pages):
            self.pools[g].give_back([p for p in pages if p >= 0])
            self._write_row(g, slot, [])
        del self._slots[slot]
        self._free_slots.append(slot)

    def _held(self, slot: int) -> _Slot:
        if slot not in self._slots:
            raise CacheError(f"slot {slot} is not held")
        return self._slots[slot]

    def live(self) -> List[int]:
        return sorted(self._slots)

    def length(self, slot: int) -> int:
        return self._held(slot).length

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    # -- pages
    def _first_needed_page(self, g: int, new_len: int, rows: int) -> int:
        """The first page a step still reads when a sequence grows to ``new_len`` by
        ``rows`` new positions: the oldest new row looks back ``window`` positions."""
        w = self.groups[g].window
        if w <= 0:
            return 0
        oldest_seen = max(0, new_len - rows + 1 - w)
        return oldest_seen // PAGE

    def reserve(self, slot: int, new_len: int, rows: int = 1) -> None:
        st = self._held(slot)
        if new_len > self.max_seq:
            raise CacheError(f"slot {slot} would reach {new_len} positions, the cache holds {self.max_seq} a sequence")
        if new_len < st.length:
            raise CacheError(f"slot {slot} holds {st.length} positions, reserve cannot shrink it to {new_len}")
        need = pages_for(new_len)
        # Count before taking, so that a refusal leaves nothing half done.
        for g, pages in enumerate(st.pages):
            more = need - len(pages)
            if more > self.pools[g].available + self._releasable(g, pages, new_len, rows):
                raise CacheError(f"the cache is full: slot {slot} needs {more} more pages of {PAGE} tokens in group {g}, "
                                 f"{self.pools[g].available} are free")
        for g, pages in enumerate(st.pages):
            first = self._first_needed_page(g, new_len, rows)
            dropped = [p for p in pages[:first] if p >= 0]
            if dropped:
                self.pools[g].give_back(dropped)
                for i in range(min(first, len(pages))):
                    pages[i] = -1
            more = need - len(pages)
            if more > 0:
                pages.extend(self.pools[g].take(more))
            if dropped or more > 0:
                self._write_row(g, slot, pages)

    def reserve_many(self, requests: Sequence[tuple]) -> None:
        """``reserve`` for several slots, all or nothing: ``requests`` holds (slot, new_len,
        rows) of distinct slots; what all of them need together is counted against every
        pool before any page moves, so a refusal leaves the bookkeeping as it was."""
        need = [0] * len(self.groups)
        for slot, new_len, rows in requests:
            st = self._held(slot)
            if new_len > self.max_seq:
                raise CacheError(f"slot {slot} would reach {new_len} positions, the cache holds {self.max_seq} a sequence")
            if new_len < st.length:
                raise CacheError(f"slot {slot} holds {st.length} positions, reserve cannot shrink it to {new_len}")
            for g, pages in enumerate(st.pages):
                need[g] += pages_for(new_len) - len(pages) - self._releasable(g, pages, new_len, rows)
        for g, n in enumerate(need):
            if n > self.pools[g].available:
                raise CacheError(f"the cache is full: this step needs {n} more pages of {PAGE} tokens in group {g}, "
                                 f"{self.pools[g].available} are free")
        for slot, new_len, rows in requests:
            self.reserve(slot, new_len, rows)

    def _releasable(self, g: int, pages: List[int], new_len: int, rows: int) -> int:
        first = self._first_needed_page(g, new_len, rows)
        return sum(1 for p in pages[:first] if p >= 0)

    def commit(self, slot: int, new_len: int) -> None:
        st = self._held(slot)
        if new_len > self.max_seq or any(pages_for(new_len) > len(pages) for pages in st.pages):
            raise CacheError(f"slot {slot}: {new_len} positions were not reserved")
        st.length = new_len

    def rollback(self, slot: int, new_len: int) -> None:
        """Cuts a sequence back to ``new_len`` positions (the reference does so by writing
        at an earlier position, crates/bc-infer/src/model.rs:321-322).  Groups that keep
        only a window may have dropped what lies before it; those refuse."""
        self.check_rollback(slot, new_len)
        st = self._held(slot)
        keep = pages_for(new_len)
        for g, pages in enumerate(st.pages):
            if len(pages) > keep:
                self.pools[g].give_back([p for p in pages[keep:] if p >= 0])
                del pages[keep:]
                self._write_row(g, slot, pages)
        st.length = new_len

    def check_rollback(self, slot: int, new_len: int) -> None:
        """Raises if ``rollback(slot, new_len)`` would be refused; changes nothing."""
        st = self._held(slot)
        if not 0 <= new_len <= st.length:
            raise CacheError(f"slot {slot} holds {st.length} positions, cannot go back to {new_len}")
        keep = pages_for(new_len)
        for g, pages in enumerate(st.pages):
            # The next row, at position new_len, looks back a window: the pages from there on must still be held.
            first = self._first_needed_page(g, new_len + 1, 1)
            if any(p < 0 for p in pages[first:keep]):
                raise CacheError(f"slot {slot}: group {g} keeps a window and no longer holds the positions before it")

    def _write_row(self, g: int, slot: int, pages: List[int]) -> None:
        row = self.tables[g][slot]
        for i in range(self.max_pages):
            row[i] = pages[i] if i < len(pages) else -1
        self.dirty.add((g, slot))

    # -- checks for tests
    def check(self) -> None:
        """Every page is free or held by exactly one slot; every slot is free or live."""
        for g, pool in enumerate(self.pools):
            seen: Dict[int, int] = {}
            for s, st in self._slots.items():
                for p in st.pages[g]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheError(f"page {p} of group {g} is held by slots {seen[p]} and {s}")
                    seen[p] = s
            if sorted(seen) != pool.held():
                raise CacheError(f"group {g}: pages held by slots {sorted(seen)} differ from the pool's {pool.held()}")
            if len(seen) + pool.available != pool.n_pages:
                raise CacheError(f"group {g}: {len(seen)} held + {pool.available} free pages are not {pool.n_pages}")
        if sorted(list(self._slots) + self._free_slots) != list(range(self.n_slots)):
            raise CacheError("a slot is lost or listed twice")
