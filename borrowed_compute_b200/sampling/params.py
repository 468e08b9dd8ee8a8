"""How the next token is picked (crates/bc-infer/src/sample.rs:11-22)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Sampling:
    """temperature <= 0 takes the highest score (greedy).  Otherwise p(i) =
    softmax(score / temperature), cut to the smallest set of tokens whose probability
    reaches ``top_p``, and drawn with a generator seeded by ``seed`` and the position of
    the row sampled, so a request can be replayed and a sequence samples the same alone or
    in any batch."""

    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if not (self.top_p > 0.0):
            raise ValueError(f"top_p must be positive, got {self.top_p}")
        if not 0 <= self.seed < (1 << 64):
            raise ValueError(f"seed must fit 64 unsigned bits, got {self.seed}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def seed_as_int64(self) -> int:
        """The seed's 64 bits as a signed integer (what an int64 tensor can hold)."""
        return self.seed - (1 << 64) if self.seed >= (1 << 63) else self.seed
