"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early,
and as many batches one after another as there are requests.

The decisions are the reference's (crates/bc-mesh/src/llm.rs:511-609): an empty prompt and
a prompt that cannot fit its answer in the context are errors (512-517); the first token
comes from the prompt's last row (535-538); a stop id ends a sequence and is not part of
its text, and so does reaching ``max_tokens`` (549-552); the loop runs while any sequence
still wants tokens (583).  What differs is that several sequences share each pass.  The
loop is written against a small backend interface so that its decisions can be tested
without a device.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

from ..sampling import RowSampler, Sampling
from .batch import StepEntry
from .engine import Engine


@dataclass
class Stats:
    """What a call cost (crates/bc-mesh/src/llm.rs:331-339): tokens in, tokens out, passes
    through the model after the prompt, and times in milliseconds."""

    prompt_tokens: int = 0
    generated: int = 0
    passes: int = 0
    first_token_ms: float = 0.0
    total_ms: float = 0.0
    first_tokens: int = 0   # tokens that came from prompt passes (one a sequence)

    @property
    def decode_tokens_per_second(self) -> float:
        """Tokens after the first over the time after the first (apps/bc-cli/src/main.rs:550-554)."""
        seconds = max(self.total_ms - self.first_token_ms, 1.0) / 1000.0
        return max(self.generated - self.first_tokens, 0) / seconds


class Backend:
    """What the loop needs of an engine.  Sequences are named by their index in the call."""

    max_batch: int = 1
    context: int = 0

    def start(self, indices: Sequence[int], prompts: Sequence[Sequence[int]], samplings: Sequence[Sampling]) -> List[int]:
        """Runs all prompts of a batch in one step; returns each sequence's first token."""
        raise NotImplementedError

    def advance(self, indices: Sequence[int], tokens: Sequence[int]) -> List[int]:
        """Feeds each live sequence its last token; returns each one's next token."""
        raise NotImplementedError

    def finish(self, index: int) -> None:
        """The sequence has ended: what it holds is given back."""
        raise NotImplementedError


def run_generation(backend: Backend, prompts: Sequence[Sequence[int]], max_tokens: int, samplings: Sequence[Sampling],
                   stop_ids: Sequence[int] = (), on_token: Optional[Callable[[int, int], None]] = None,
                   clock: Callable[[], float] = time.perf_counter) -> tuple:
    """Generates up to ``max_tokens`` after each prompt.  Returns (tokens per prompt, Stats)."""
    if len(samplings) != len(prompts):
        raise ValueError("one Sampling per prompt")
    if max_tokens < 0:
        raise ValueError("max_tokens cannot be negative")
    for p in prompts:
        if len(p) == 0:
            raise ValueError("the prompt is empty")
        if backend.context and len(p) + max_tokens > backend.context:
            raise ValueError(f"{len(p)} prompt tokens plus {max_tokens} to write exceed the context of {backend.context}")
    stops = set(int(s) for s in stop_ids)
    out: List[List[int]] = [[] for _ in prompts]
    stats = Stats(prompt_tokens=sum(len(p) for p in prompts))
    started = clock()

    def push(i: int, tok: int) -> bool:
        """Takes a token for sequence i; False once the sequence has ended."""
        if tok in stops or len(out[i]) >= max_tokens:
            return False
        out[i].append(tok)
        if on_token is not None:
            on_token(i, tok)
        return len(out[i]) < max_tokens

    order = list(range(len(prompts)))
    for at in range(0, len(order), max(1, backend.max_batch)):
        batch = order[at:at + max(1, backend.max_batch)]
        first = backend.start(batch, [prompts[i] for i in batch], [samplings[i] for i in batch])
        if at == 0:
            stats.first_token_ms = (clock() - started) * 1000.0
        stats.first_tokens += len(batch)
        live = []
        for i, tok in zip(batch, first):
            if push(i, int(tok)):
                live.append(i)
            else:
                backend.finish(i)
        while live:
            stats.passes += 1
            nxt = backend.advance(live, [out[i][-1] for i in live])
            still = []
            for i, tok in zip(live, nxt):
                if push(i, int(tok)):
                    still.append(i)
                else:
                    backend.finish(i)
            live = still
    stats.generated = sum(len(o) for o in out)
    stats.total_ms = (clock() - started) * 1000.0
    return out, stats


class EngineBackend(Backend):
    """Drives an Engine: one slot a sequence, scores sampled on the device, token ids read
    back to the host once a step."""

    def __init__(self, engine: Engine, max_batch: Optional[int] = None):
        self.engine = engine
        self.max_batch = max_batch or engine.cache.slots.n_slots
        self.context = engine.max_seq
        self.sampler = RowSampler(engine.rt.device, self.max_batch)
        self._slot = {}
        self._sampling = {}
        self._live_key = None
        self._steps = torch.zeros(self.max_batch, dtype=torch.int32, device=engine.rt.device)
        self._host_steps = torch.zeros(self.max_batch, dtype=torch.int32).pin_memory()

    def _set_rows(self, indices: Sequence[int]) -> None:
        key = tuple(indices)
        if key != self._live_key:
            self.sampler.set_rows([self._sampling[i] for i in indices])
            self._live_key = key

    def _sample(self, scores: torch.Tensor, positions: Sequence[int]) -> List[int]:
        if not self.sampler.all_greedy:      # only a draw needs to know the position it is for
            n = len(positions)
            self._host_steps[:n] = torch.tensor(positions, dtype=torch.int32)
            self._steps[:n].copy_(self._host_steps[:n], non_blocking=True)
        ids = self.sampler.sample(scores, self._steps).tolist()   # the step's one synchronisation with the device
        self.engine.raise_on_kernel_error()
        return ids

    def start(self, indices, prompts, samplings) -> List[int]:
        entries = []
        try:
            for i, p, s in zip(indices, prompts, samplings):
                self._slot[i] = self.engine.acquire()
                self._sampling[i] = s
                entries.append(StepEntry(self._slot[i], list(p), want=(len(p) - 1,)))
            self._set_rows(indices)
            scores = self.engine.step(entries)
        except Exception:
            for i in indices:
                if i in self._slot:
                    self.finish(i)
            raise
        # The draw's step is the position of the row sampled (crates/bc-mesh/src/engine.rs:347-350).
        return self._sample(scores, [len(p) - 1 for p in prompts])

    def advance(self, indices, tokens) -> List[int]:
        entries = [StepEntry(self._slot[i], (int(t),), want=(0,)) for i, t in zip(indices, tokens)]
        positions = [self.engine.length(self._slot[i]) for i in indices]
        self._set_rows(indices)
        scores = self.engine.step(entries, borrow_scores=True)   # sampled from at once, below
        return self._sample(scores, positions)

    def finish(self, index: int) -> None:
        self.engine.release(self._slot.pop(index))
        self._sampling.pop(index, None)
        self._live_key = None
