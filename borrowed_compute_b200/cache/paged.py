"""The cache on the device: pages of keys and values per storage group, page tables that
mirror the host's bookkeeping, and per-sequence state of fixed size.

Runs of layers whose mixers need the same memory (the same planes of values a position,
the same window) form one *group* with storage of its own:

    planes[i]  [runs in the group, pages, heads_i, 64, width_i]   (keys and values are two planes)
    table      [slots, pages a sequence can have] int32, -1 where no page is held

A mixer that asks for state gets one tensor [slots, *shape] for its run, zeroed whenever a
slot is handed out.  The reference's cache is one f32 buffer per layer and conversation
(crates/bc-infer/src/gpu/mod.rs:294-342).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, RunMemory, Runtime, StateNeed
from .slots import PAGE, GroupPlan, SlotTable, pages_for


@dataclass
class _Group:
    need: CacheNeed
    runs: List[int]                 # schedule entries that own a line of this group
    planes: Optional[List[torch.Tensor]] = None
    table: Optional[torch.Tensor] = None
    host_table: Optional[torch.Tensor] = None


class PagedCache:
    """Storage for every run of a model's schedule, sized by tokens, slots and the longest
    sequence.  ``needs[i]`` / ``states[i]`` are what run i's mixer asked for (or None);
    ``memory_of[i]`` names the run whose memory run i reads instead of owning some."""

    def __init__(self, rt: Runtime, needs: Sequence[Optional[CacheNeed]], states: Sequence[Optional[StateNeed]],
                 memory_of: Sequence[Optional[int]], max_tokens: int, n_slots: int, max_seq: int):
        self.rt = rt
        self.n_runs = len(needs)
        self.memory_of = list(memory_of)
        self.groups: List[_Group] = []
        self._line: Dict[int, Tuple[int, int]] = {}      # owning run -> (group, line)
        by_key: Dict[Tuple, int] = {}
        for i, need in enumerate(needs):
            if need is None or self.memory_of[i] is not None:
                continue
            g = by_key.setdefault(need.key(), len(self.groups))
            if g == len(self.groups):
                self.groups.append(_Group(need, []))
            self._line[i] = (g, len(self.groups[g].runs))
            self.groups[g].runs.append(i)
        n_pages = max(1, pages_for(max_tokens))
        self.n_pages = n_pages
        self.slots = SlotTable(n_slots, n_pages, max_seq, [GroupPlan(g.need.window) for g in self.groups])
        for g in self.groups:
            g.planes = [torch.zeros((len(g.runs), n_pages, heads, PAGE, width), dtype=rt.dtype, device=rt.device)
                        for heads, width in g.need.planes]
            g.host_table = torch.full((n_slots, self.slots.max_pages), -1, dtype=torch.int32).pin_memory() \
                if rt.device.type == "cuda" else torch.full((n_slots, self.slots.max_pages), -1, dtype=torch.int32)
            g.table = torch.full((n_slots, self.slots.max_pages), -1, dtype=torch.int32, device=rt.device)
        self._copied: Optional[torch.cuda.Event] = None
        self.state: Dict[int, torch.Tensor] = {}
        for i, need in enumerate(states):
            if need is not None and self.memory_of[i] is None:
                self.state[i] = torch.zeros((n_slots,) + tuple(need.shape), dtype=need.dtype, device=rt.device)

    # -- slots
    def acquire(self) -> int:
        slot = self.slots.acquire()
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.slots.release(slot)

    def sync_tables(self) -> int:
        """Brings the device page tables up to date with the host's bookkeeping; returns
        the bytes copied to the device."""
        if not self.slots.dirty:
            return 0
        touched = set()
        if self._copied is not None:
            self._copied.synchronize()   # the last copy out of the pinned tables is done
        for g, slot in self.slots.dirty:
            self.groups[g].host_table[slot] = torch.tensor(self.slots.tables[g][slot], dtype=torch.int32)
            touched.add(g)
        self.slots.dirty.clear()
        for g in touched:
            self.groups[g].table.copy_(self.groups[g].host_table, non_blocking=True)
        if self.rt.device.type == "cuda":
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()
        return sum(self.groups[g].host_table.numel() * 4 for g in touched)

    # -- what a run sees
    def memory(self, run: int) -> RunMemory:
        owner = run if self.memory_of[run] is None else self.memory_of[run]
        mem = RunMemory(writes=self.memory_of[run] is None)
        if owner in self._line:
            g, line = self._line[owner]
            grp = self.groups[g]
            mem.planes, mem.page_table = tuple(t[line] for t in grp.planes), grp.table
        if owner in self.state:
            mem.state = self.state[owner]
        return mem

    def bytes(self) -> int:
        total = sum(t.numel() * t.element_size() for g in self.groups for t in g.planes)
        return total + sum(t.numel() * t.element_size() for t in self.state.values())

    def bytes_per_token(self) -> int:
        return sum(len(g.runs) * g.need.values_per_token() * g.planes[0].element_size() for g in self.groups)
