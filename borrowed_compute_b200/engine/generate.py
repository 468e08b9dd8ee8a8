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
from .engine import Engine, count_traffic


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


class Pending:
    """The token ids of a step that may still be running on the device."""

    def ids(self) -> List[int]:
        """Waits for the step and returns one id a sequence of the step, in its order."""
        raise NotImplementedError


class _Ready(Pending):
    def __init__(self, ids: Sequence[int]):
        self._ids = [int(t) for t in ids]

    def ids(self) -> List[int]:
        return self._ids


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

    def begin(self, indices: Sequence[int], tokens: Optional[Sequence[int]]) -> Optional[Pending]:
        """Starts ``advance`` without waiting for its ids.  ``tokens`` None asks for a step
        that follows the step begun last for exactly these sequences, each fed the id that
        step samples for it, whether or not the host has read that id yet; a backend that
        cannot do so (now, or ever) returns None and the loop reads the ids first.  The
        default is ``advance`` itself: nothing overlaps."""
        return None if tokens is None else _Ready(self.advance(indices, tokens))

    def finish(self, index: int) -> None:
        """The sequence has ended: what it holds is given back."""
        raise NotImplementedError


def run_generation(backend: Backend, prompts: Sequence[Sequence[int]], max_tokens: int, samplings: Sequence[Sampling],
                   stop_ids: Sequence[int] = (), on_token: Optional[Callable[[int, int], None]] = None,
                   clock: Callable[[], float] = time.perf_counter, include_stop: bool = False) -> tuple:
    """Generates up to ``max_tokens`` after each prompt.  Returns (tokens per prompt, Stats).
    A stop id ends its sequence and is left out of it, or, with ``include_stop``, is its last
    id (counted against ``max_tokens`` like any other)."""
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
        if len(out[i]) >= max_tokens or (tok in stops and not include_stop):
            return False
        out[i].append(tok)
        if tok in stops:
            if on_token is not None:
                on_token(i, tok)
            return False
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
        # One token a live sequence a pass.  Where the backend can, the next pass is begun
        # before this one's ids are read (it is fed them on the device), so the device never
        # waits for the host; the host then learns one pass late that a stop id came, and
        # that sequence's row of the pass in flight has run for nothing.  A pass that would be
        # a sequence's last by count is never run ahead of.
        pending = backend.begin(live, [out[i][-1] for i in live]) if live else None
        dead: set = set()      # sequences of the pass in flight that had ended before it began
        while pending is not None:
            ahead = None
            if not dead and all(len(out[i]) + 1 < max_tokens for i in live):
                ahead = backend.begin(live, None)
            ids = pending.ids()
            stats.passes += 1
            ended = set()
            for i, tok in zip(live, ids):
                if i not in dead and not push(i, int(tok)):
                    ended.add(i)
            if ahead is not None:
                pending, dead = ahead, ended
                continue
            for i in live:
                if i in dead or i in ended:
                    backend.finish(i)
            live = [i for i in live if i not in dead and i not in ended]
            dead = set()
            pending = backend.begin(live, [out[i][-1] for i in live]) if live else None
    stats.generated = sum(len(o) for o in out)
    stats.total_ms = (clock() - started) * 1000.0
    return out, stats


class _OnDevice(Pending):
    """Ids on their way to pinned host memory; ``ids`` waits for that copy alone."""

    def __init__(self, host: torch.Tensor, n: int, copied: torch.cuda.Event, engine: Engine):
        self.host, self.n, self.copied, self.engine = host, n, copied, engine

    def ids(self) -> List[int]:
        self.copied.synchronize()                 # the pass's one synchronisation with the device
        self.engine.raise_on_kernel_error()
        return self.host[: self.n].tolist()


class EngineBackend(Backend):
    """Drives an Engine: one slot a sequence, scores sampled on the device, token ids copied
    to pinned host memory once a pass.  On the captured decode path the sampler writes each
    id straight into the next pass's token buffer, so the next pass can be launched before
    the host has seen the ids."""

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
        self._host_ids = [torch.zeros(self.max_batch, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._copied = [torch.cuda.Event(), torch.cuda.Event()]
        self._flip = 0

    def _set_rows(self, indices: Sequence[int]) -> None:
        key = tuple(indices)
        if key != self._live_key:
            self.sampler.set_rows([self._sampling[i] for i in indices])
            self._live_key = key

    def _sample(self, scores: torch.Tensor, positions: Sequence[int], decode: bool = True) -> Pending:
        """Samples one id a row.  The draw's step is the position of the row sampled
        (crates/bc-mesh/src/engine.rs:347-350)."""
        n = scores.shape[0]
        graph = self.engine.last_graph
        if graph is not None:
            # A captured decode step: its rows' positions are on the device already, and the ids
            # go where the next pass of the same sequences reads its tokens.
            ids = self.sampler.sample(scores, graph.views["row_pos"], out=graph.views["tokens"][:n])
        else:
            if not self.sampler.all_greedy:      # only a draw needs to know the position it is for
                self._host_steps[:n] = torch.tensor(positions, dtype=torch.int32)
                self._steps[:n].copy_(self._host_steps[:n], non_blocking=True)
                count_traffic("h2d", 4 * n, decode)
            ids = self.sampler.sample(scores, self._steps)
        self._flip ^= 1
        host, copied = self._host_ids[self._flip], self._copied[self._flip]
        host[:n].copy_(ids, non_blocking=True)
        copied.record()
        count_traffic("d2h", 4 * n, decode)
        return _OnDevice(host, n, copied, self.engine)

    def start(self, indices, prompts, samplings) -> List[int]:
        entries = []
        try:
            for i, p, s in zip(indices, prompts, samplings):
                self._slot[i] = self.engine.acquire()
                self._sampling[i] = s
                entries.append(StepEntry(self._slot[i], list(p), want=(len(p) - 1,)))
            self._set_rows(indices)
            scores = self.engine.step(entries, borrow_scores=True)
        except Exception:
            for i in indices:
                if i in self._slot:
                    self.finish(i)
            raise
        return self._sample(scores, [len(p) - 1 for p in prompts], decode=False).ids()

    def begin(self, indices, tokens) -> Optional[Pending]:
        slots = [self._slot[i] for i in indices]
        self._set_rows(indices)
        if tokens is None:
            if not self.engine.can_step_again(slots):
                return None
            positions = [self.engine.length(s) for s in slots]
            scores = self.engine.step_again(borrow_scores=True)
        else:
            positions = [self.engine.length(s) for s in slots]
            scores = self.engine.step([StepEntry(s, (int(t),), want=(0,)) for s, t in zip(slots, tokens)], borrow_scores=True)
        return self._sample(scores, positions)

    def advance(self, indices, tokens) -> List[int]:
        return self.begin(indices, tokens).ids()

    def finish(self, index: int) -> None:
        self.engine.release(self._slot.pop(index))
        self._sampling.pop(index, None)
        self._live_key = None
