"""Sampling on the device: per-row parameters in tensors, one fused kernel a batch."""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from .params import Sampling


class RowSampler:
    """Holds the per-row parameter tensors of a batch, so that successive steps of the
    same batch reuse them (and a captured graph can read them in place)."""

    def __init__(self, device: torch.device, capacity: int):
        self.capacity = capacity
        self.temperature = torch.zeros(capacity, dtype=torch.float32, device=device)
        self.top_p = torch.ones(capacity, dtype=torch.float32, device=device)
        self.seed = torch.zeros(capacity, dtype=torch.int64, device=device)
        self.out = torch.zeros(capacity, dtype=torch.int32, device=device)
        self.all_greedy = True

    def set_rows(self, samplings: Sequence[Sampling]) -> None:
        n = len(samplings)
        if n > self.capacity:
            raise ValueError(f"{n} rows exceed the sampler's {self.capacity}")
        self.all_greedy = all(s.greedy for s in samplings)
        self.temperature[:n].copy_(torch.tensor([s.temperature for s in samplings], dtype=torch.float32))
        self.top_p[:n].copy_(torch.tensor([s.top_p for s in samplings], dtype=torch.float32))
        self.seed[:n].copy_(torch.tensor([s.seed_as_int64 for s in samplings], dtype=torch.int64))

    def sample(self, scores: torch.Tensor, step: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Token ids [rows] int32 for scores [rows, vocab]; ``step[r]`` is the position of
        the row sampled (crates/bc-mesh/src/engine.rs:347-350).  The ids go to ``out`` if
        given (int32, at least ``rows`` long), else to a buffer of this sampler's."""
        rows = scores.shape[0]
        out = self.out[:rows] if out is None else out[:rows]
        if self.all_greedy:
            ops.argmax(scores, out)
        else:
            ops.sample(scores, self.temperature, self.top_p, self.seed, step, out)
        return out
