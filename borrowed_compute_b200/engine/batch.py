"""Flattening one step's sequences into rows.

A step brings, for each sequence, its next tokens (a whole prompt, or one token).  All
products, norms and the feed-forward run on the rows of all sequences at once; only the
mixer needs to know which row belongs to which sequence and where.  The reference feeds
one sequence a pass and gives each row a position (crates/bc-infer/src/model.rs:411-425);
this is the same idea across sequences.  Planning is host-only code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class StepEntry:
    """One sequence's share of a step: the slot it lives in, its next tokens, and the
    indices among these tokens whose scores are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepPlan:
    rows: int
    seqs: int
    padded_rows: int
    tokens: np.ndarray      # [padded_rows] int32
    row_pos: np.ndarray     # [padded_rows] int32
    row_slot: np.ndarray    # [padded_rows] int32, -1 on padding
    seq_rows: np.ndarray    # [seqs + 1] int32
    seq_slot: np.ndarray    # [seqs] int32
    seq_start: np.ndarray   # [seqs] int32
    want_rows: np.ndarray   # [n_want] int32, in entry order then want order
    max_new: int
    max_total: int
    decode: bool

    def packed(self) -> np.ndarray:
        """All arrays in one int32 vector, in the order of ``layout``."""
        return np.concatenate([self.tokens, self.row_pos, self.row_slot, self.seq_rows, self.seq_slot, self.seq_start, self.want_rows])

    def layout(self) -> List[Tuple[str, int]]:
        return [("tokens", self.padded_rows), ("row_pos", self.padded_rows), ("row_slot", self.padded_rows),
                ("seq_rows", self.seqs + 1), ("seq_slot", self.seqs), ("seq_start", self.seqs), ("want_rows", len(self.want_rows))]


def plan_step(entries: Sequence[StepEntry], starts: Sequence[int], pad_rows_to: int = 1) -> StepPlan:
    """``starts[i]`` is how many positions entry i's slot already holds.  Rows are padded
    up to a multiple of ``pad_rows_to`` with rows that belong to no sequence."""
    if not entries:
        raise ValueError("a step needs at least one sequence")
    if len(entries) != len(starts):
        raise ValueError("one start per entry")
    counts = [len(e.tokens) for e in entries]
    if min(counts) <= 0:
        raise ValueError("every sequence of a step brings at least one token")
    if len({e.slot for e in entries}) != len(entries):
        raise ValueError("a slot appears twice in one step")
    rows = sum(counts)
    padded = -(-rows // pad_rows_to) * pad_rows_to
    tokens = np.zeros(padded, dtype=np.int32)
    row_pos = np.zeros(padded, dtype=np.int32)
    row_slot = np.full(padded, -1, dtype=np.int32)
    seq_rows = np.zeros(len(entries) + 1, dtype=np.int32)
    want: List[int] = []
    r = 0
    for i, (e, start) in enumerate(zip(entries, starts)):
        n = counts[i]
        tokens[r:r + n] = np.asarray(e.tokens, dtype=np.int64)
        row_pos[r:r + n] = np.arange(start, start + n, dtype=np.int32)
        row_slot[r:r + n] = e.slot
        for w in e.want:
            if not 0 <= w < n:
                raise ValueError(f"wanted index {w} is outside the {n} tokens of slot {e.slot}")
            want.append(r + int(w))
        r += n
        seq_rows[i + 1] = r
    return StepPlan(
        rows=rows, seqs=len(entries), padded_rows=padded, tokens=tokens, row_pos=row_pos, row_slot=row_slot, seq_rows=seq_rows,
        seq_slot=np.asarray([e.slot for e in entries], dtype=np.int32), seq_start=np.asarray(starts, dtype=np.int32),
        want_rows=np.asarray(want, dtype=np.int32), max_new=max(counts), max_total=max(s + n for s, n in zip(starts, counts)),
        decode=all(n == 1 for n in counts))
