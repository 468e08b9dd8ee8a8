"""The engine: a loaded model, its cache, and the one step function everything runs through.

``step`` takes a batch of sequences that either all start (their prompts, of unequal
lengths, in one step) or all go on, runs exactly the tokens it is given as one batch
against what earlier steps left in the cache, and returns float32 scores at the wanted
places.  Generation, trace replay and the benchmark all call it.  The reference's
counterpart feeds one sequence a call (crates/bc-mesh/src/engine.rs:287-363;
crates/bc-infer/src/model.rs:285-352) and guards the same things: positions may not skip
(model.rs:303-305), the context may not overflow (306-308), tokens must lie in the
vocabulary (274-276).
"""

from __future__ import annotations

import gc
import weakref

from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache import PAGE, PagedCache
from ..config.errors import CacheError
from ..parts.base import Runtime, StepContext
from ..weights import TensorSource, load_tensors, random_tensors, read_config_json, read_generation_stop_ids
from .batch import StepEntry, StepPlan, plan_step
from .model import DecoderModel, model_for_config

# Bytes copied between host and device since import, counted where the copies are issued
# (the benchmark reports them per step): all of them, and those of decode steps alone.
TRAFFIC = {"h2d": 0, "d2h": 0, "h2d_decode": 0, "d2h_decode": 0}


def count_traffic(direction: str, n_bytes: int, decode: bool) -> None:
    TRAFFIC[direction] += n_bytes
    if decode:
        TRAFFIC[direction + "_decode"] += n_bytes


DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class _DecodeGraph:
    """One captured decode step for a fixed number of rows, none of which reaches past
    ``reach`` positions (parts may plan by that bound: the decode attention cuts long
    sequences into more pieces)."""

    def __init__(self, engine: "Engine", rows: int, reach: int):
        self._engine, self.rows, self.reach = weakref.ref(engine), rows, reach   # no cycle: a dropped engine and its graphs go at once
        dev = engine.rt.device
        # tokens, row_pos, row_slot, seq_rows (+1), seq_slot, seq_start, want_rows
        self.sizes = [("tokens", rows), ("row_pos", rows), ("row_slot", rows), ("seq_rows", rows + 1), ("seq_slot", rows),
                      ("seq_start", rows), ("want_rows", rows)]
        total = sum(n for _, n in self.sizes)
        self.ints = torch.zeros(total, dtype=torch.int32, device=dev)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.copied: Optional[torch.cuda.Event] = None
        self.views, at = {}, 0
        for name, n in self.sizes:
            self.views[name] = self.ints[at:at + n]
            at += n
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.scores: Optional[torch.Tensor] = None

    def pack(self, tokens, row_pos, row_slot, rows_used: int) -> np.ndarray:
        """The step's integers in the layout of ``sizes``: one row a sequence, padding rows
        (slot -1) after them.  ``tokens`` may be None and filled into [:rows_used] later."""
        rows, n = self.rows, rows_used
        out = np.zeros(sum(size for _, size in self.sizes), dtype=np.int32)
        at = {}
        o = 0
        for name, size in self.sizes:
            at[name] = o
            o += size
        if tokens is not None:
            out[at["tokens"]:at["tokens"] + n] = tokens
        out[at["row_pos"]:at["row_pos"] + n] = row_pos
        out[at["row_slot"]:at["row_slot"] + rows] = -1
        out[at["row_slot"]:at["row_slot"] + n] = row_slot
        out[at["seq_rows"]:at["seq_rows"] + rows + 1] = n
        out[at["seq_rows"]:at["seq_rows"] + n + 1] = np.arange(n + 1, dtype=np.int32)
        out[at["seq_slot"]:at["seq_slot"] + rows] = -1
        out[at["seq_slot"]:at["seq_slot"] + n] = row_slot
        out[at["seq_start"]:at["seq_start"] + n] = row_pos
        out[at["want_rows"]:at["want_rows"] + rows] = np.arange(rows, dtype=np.int32)
        return out

    def _upload(self, packed: np.ndarray, keep_tokens: bool = False) -> None:
        """Sends the step's integers; with ``keep_tokens`` all but the tokens, which then stay
        as something on the device (the last step's sampler) left them."""
        if self.copied is not None:
            self.copied.synchronize()   # the last copy out of the pinned buffer is done
        first = self.rows if keep_tokens else 0     # the tokens come first in the layout
        self.host[first:].copy_(torch.from_numpy(packed[first:]))
        self.ints[first:].copy_(self.host[first:], non_blocking=True)
        count_traffic("h2d", 4 * (self.host.numel() - first), True)
        if self.copied is None:
            self.copied = torch.cuda.Event()
        self.copied.record()

    @property
    def engine(self) -> "Engine":
        eng = self._engine()
        if eng is None:
            raise RuntimeError("the engine of this captured step is gone")
        return eng

    def _forward(self) -> torch.Tensor:
        v, rows = self.views, self.rows
        ctx = StepContext(rows=rows, seqs=rows, tokens=v["tokens"], row_pos=v["row_pos"], row_slot=v["row_slot"], seq_rows=v["seq_rows"],
                          seq_slot=v["seq_slot"], seq_start=v["seq_start"], max_new=1, max_total=self.reach, decode=True,
                          extras={"graph": True})
        return self.engine.model.forward(ctx, self.engine.cache, v["want_rows"], rows)

    def run(self, packed: np.ndarray, keep_tokens: bool = False) -> torch.Tensor:
        if self.graph is None:
            # Warm-up and capture run on padding rows only (every slot -1), which change nothing
            # that outlives the step: the real rows then run exactly once, in the replay below.
            # A mixer that keeps state of its own would otherwise see its first step twice.
            self._upload(self.pack(None, [], [], 0))
            self._forward()   # once eagerly: first-use set-up must not happen inside a capture
            torch.cuda.synchronize()
            # Nothing may free device memory or destroy another graph while this one is being
            # captured: objects waiting for the cycle collector (an engine dropped earlier in
            # the process, with its graphs) go now, and the collector rests during the capture.
            gc.collect()
            was_enabled = gc.isenabled()
            gc.disable()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self.scores = self._forward()
            finally:
                if was_enabled:
                    gc.enable()
            self.graph = graph
        self._upload(packed, keep_tokens)
        self.graph.replay()
        return self.scores


class _Ahead:
    """The next decode step of the same sequences, staged on the host while the device
    still runs the current one: slots reserved, page tables sent, every integer of the
    step but the tokens."""

    def __init__(self, slots, starts, graph: _DecodeGraph, packed: np.ndarray):
        self.slots, self.starts, self.graph, self.packed = tuple(slots), list(starts), graph, packed


class Engine:
    def __init__(self, config: Mapping[str, Any], model: DecoderModel, typed_config: Any, rt: Runtime, max_tokens: int,
                 max_slots: int, max_seq: int):
        self.config, self.model, self.typed_config, self.rt = dict(config), model, typed_config, rt
        self.vocab_size = model.spec.vocab_size
        self.max_seq = max_seq
        self.stop_ids: tuple = tuple(model.spec.stop_ids)    # ids that end a sequence by default: config.json's, plus generation_config.json's
        needs, states, memory_of = model.memory_needs()
        self.cache = PagedCache(rt, needs, states, memory_of, max_tokens=max_tokens, n_slots=max_slots, max_seq=max_seq)
        self._ints: Optional[torch.Tensor] = None
        self._host_ints: Optional[torch.Tensor] = None
        self._staged: Optional[torch.cuda.Event] = None
        self._graphs: Dict[Tuple[int, int], "_DecodeGraph"] = {}
        self._ahead: Optional[_Ahead] = None
        self.last_graph: Optional[_DecodeGraph] = None   # the captured step the last call of step() replayed, if it did
        # Decode steps replay a captured CUDA graph unless a part plans on the host.
        self.use_graphs = all(part.graph_safe for _, part in model.named_parts()) and not ops.bounds_check
        self.steps_run = 0

    # ------------------------------------------------------------------------ construction
    @staticmethod
    def _runtime(dtype, device) -> Runtime:
        if dtype not in DTYPES:
            raise ValueError(f"dtype {dtype!r} is neither bfloat16 nor float32")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError(f"the engine runs on a CUDA device only, not on {dev}")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; there is no CPU path")
        ops.lib()  # fail now, and loudly, if the kernels cannot be had
        with torch.cuda.device(dev):
            ops.bind_status(dev)
            ops.self_check(dev)   # once a device: every product against float64 sums, before anything is trusted to it
        return Runtime(device=dev, dtype=DTYPES[dtype])

    @classmethod
    def _sized(cls, config, model, typed, rt, max_tokens, max_slots, max_seq) -> "Engine":
        limit = model.spec.max_positions
        max_seq = min(limit, max_seq) if max_seq else min(limit, 8192)
        if max_tokens is None:
            max_tokens = min(max_seq * (max_slots or 8), 1 << 17)
        max_tokens = -(-int(max_tokens) // PAGE) * PAGE
        max_seq = min(max_seq, max_tokens)
        if max_slots is None:
            max_slots = max(1, min(max_tokens // PAGE, 1024))
        rt.max_positions = max_seq
        return cls(config, model, typed, rt, max_tokens, max_slots, max_seq)

    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", max_tokens: Optional[int] = None,
                    max_slots: Optional[int] = None, max_seq: Optional[int] = None, progress=None) -> "Engine":
        """Loads ``config.json`` and the safetensors of a model folder; ``progress(done,
        total)`` is called after every tensor brought to the device (the reference reports
        bytes fetched as it goes, crates/bc-infer/src/lib.rs:33-47)."""
        config = read_config_json(folder)
        typed, model = model_for_config(config)
        rt = cls._runtime(dtype, device)
        eng = cls._sized(config, model, typed, rt, max_tokens, max_slots, max_seq)
        model.load(load_tensors(model.expected_tensors(), TensorSource(folder), rt, progress), rt)
        more = read_generation_stop_ids(folder, eng.vocab_size)
        eng.stop_ids = tuple(dict.fromkeys(eng.stop_ids + more))
        return eng

    @classmethod
    def from_random(cls, config: Mapping[str, Any], seed: int, dtype="bfloat16", device="cuda:0",
                    max_tokens: Optional[int] = None, max_slots: Optional[int] = None, max_seq: Optional[int] = None,
                    stored_dtype=None) -> "Engine":
        """Random weights drawn on the device, without a folder: the same values, to the
        bit, as a folder written from the same configuration and seed holds.  ``stored_dtype``
        is the type that folder would store (default: ``dtype``); a float32 engine over
        values stored as bfloat16 is what the plain implementation is compared with."""
        from ..weights.loader import device_type

        typed, model = model_for_config(config)
        rt = cls._runtime(dtype, device)
        stored = rt.dtype if stored_dtype is None else DTYPES[stored_dtype]
        eng = cls._sized(config, model, typed, rt, max_tokens, max_slots, max_seq)
        tensors = {}
        for name, spec in model.expected_tensors().items():
            if spec.optional:
                continue
            t = random_tensors({name: spec}, seed, stored, rt.device)[name]
            tensors[name] = t.to(device_type(spec, t.dtype, rt))
        model.load(tensors, rt)
        return eng

    @classmethod
    def from_tensors(cls, config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], dtype="bfloat16", device="cuda:0",
                     max_tokens: Optional[int] = None, max_slots: Optional[int] = None, max_seq: Optional[int] = None) -> "Engine":
        """Tensors given by name in memory, checked like a folder's."""
        from ..weights.loader import check_tensors, device_type

        typed, model = model_for_config(config)
        rt = cls._runtime(dtype, device)
        eng = cls._sized(config, model, typed, rt, max_tokens, max_slots, max_seq)
        expected = model.expected_tensors()
        check_tensors(expected, {n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()}, "the given tensors")
        model.load({n: tensors[n].to(device=rt.device, dtype=device_type(s, tensors[n].dtype, rt)).contiguous()
                    for n, s in expected.items() if n in tensors}, rt)
        return eng

    # ------------------------------------------------------------------------------- slots
    def acquire(self) -> int:
        """A slot for a new sequence; its state is zero and it holds no positions."""
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        """Gives a sequence's slot and pages back."""
        self._ahead = None
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.slots.length(slot)

    def rollback(self, slot: int, length: int) -> None:
        """Cuts a sequence back to ``length`` positions; the next step writes from there.

        Token-indexed memory goes back by its length.  Per-sequence state has already
        absorbed the dropped positions: a cut to 0 clears it (that is the state of a new
        sequence); any other cut asks each mixer that keeps state to restore it
        (``Mixer.rollback_state``) and is refused with a CacheError, leaving everything as it
        was, unless all of them can."""
        self._ahead = None
        have = self.cache.slots.length(slot)
        if not 0 <= length <= have:
            raise CacheError(f"slot {slot} holds {have} positions, cannot go back to {length}")
        if length == have:
            return
        self.cache.slots.check_rollback(slot, length)
        saved = {run: state[slot].clone() for run, state in self.cache.state.items()}
        for run, state in self.cache.state.items():
            if length == 0:
                state[slot].zero_()
                continue
            mixer = self.model.blocks[self.model.spec.schedule[run].layer].memory_part()
            if not mixer.rollback_state(state, slot, length):
                for r, old in saved.items():
                    self.cache.state[r][slot].copy_(old)
                raise CacheError(f"slot {slot} cannot go back to {length} positions: the mixer of run {run} keeps per-sequence "
                                 f"state and cannot restore it (only a cut to 0 is always possible)")
        self.cache.slots.rollback(slot, length)

    # -------------------------------------------------------------------------------- step
    def _stage(self, plan: StepPlan) -> Dict[str, torch.Tensor]:
        packed = plan.packed()
        n = packed.size
        if self._ints is None or self._ints.numel() < n:
            cap = max(4096, 2 * n)
            self._ints = torch.empty(cap, dtype=torch.int32, device=self.rt.device)
            self._host_ints = torch.empty(cap, dtype=torch.int32).pin_memory()
            self._staged = None
        if self._staged is not None:
            self._staged.synchronize()   # the last copy out of the pinned buffer is done
        self._host_ints[:n].copy_(torch.from_numpy(packed))
        self._ints[:n].copy_(self._host_ints[:n], non_blocking=True)
        count_traffic("h2d", 4 * n, plan.decode)
        if self._staged is None:
            self._staged = torch.cuda.Event()
        self._staged.record()
        views, at = {}, 0
        for name, size in plan.layout():
            views[name] = self._ints[at:at + size]
            at += size
        return views

    def check_entries(self, entries: Sequence[StepEntry]) -> List[int]:
        """The guards of a step; returns every entry's start position."""
        starts = []
        for e in entries:
            start = self.cache.slots.length(e.slot)   # raises if the slot is not held
            if len(e.tokens) == 0:
                raise ValueError(f"slot {e.slot} brings no tokens")
            if start + len(e.tokens) > self.max_seq:
                raise CacheError(f"{start + len(e.tokens)} tokens are past the {self.max_seq} positions a sequence can hold")
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise ValueError(f"token {t} is outside the vocabulary")
            starts.append(start)
        return starts

    # ------------------------------------------------------------------------ decode graphs
    @staticmethod
    def _bucket(n: int) -> int:
        """Rows a captured decode step is padded to: a power of two up to 16, then
        multiples of 16 (the smallest token tile of the tensor-core product)."""
        b = 1
        while b < n and b < 16:
            b *= 2
        return b if n <= 16 else -(-n // 16) * 16

    def _reach(self, total: int) -> int:
        """The bound on positions that a captured step is made for: ``total`` rounded up to a
        power of two from 4,096 on, at most what a sequence can hold."""
        reach = 4096
        while reach < total:
            reach *= 2
        return min(reach, self.max_seq)

    def _graph_for(self, n: int, total: int) -> _DecodeGraph:
        """The captured step for ``n`` sequences of which the longest reaches ``total`` positions."""
        key = (self._bucket(n), self._reach(total))
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _DecodeGraph(self, *key)
        return g

    def can_step_again(self, slots: Sequence[int]) -> bool:
        """Whether ``step_again`` can follow now: the last step was a captured decode step of
        exactly these slots, in this order, and the step after it is staged."""
        a = self._ahead
        return a is not None and self.last_graph is a.graph and a.slots == tuple(slots) and \
            all(self.cache.slots.length(s) == p for s, p in zip(a.slots, a.starts))

    def step_again(self, borrow_scores: bool = False) -> torch.Tensor:
        """One more token for exactly the sequences of the last (captured) decode step, each
        fed the id that lies at its row of ``last_graph.views["tokens"]`` on the device:
        whoever sampled from the last step's scores wrote it there, and the host need not
        have seen it.  Check ``can_step_again`` first."""
        a = self._ahead
        if a is None or self.last_graph is not a.graph:
            raise RuntimeError("no staged step to go on from: the last step was not a captured decode step")
        return self._decode_graph_step([StepEntry(s, (0,), want=(0,)) for s in a.slots], borrow_scores, tokens_on_device=True)

    def _decode_graph_step(self, entries: Sequence[StepEntry], borrow_scores: bool, tokens_on_device: bool = False) -> torch.Tensor:
        """A step of one token a sequence, replayed from a CUDA graph captured once per
        padded batch size: the kernels, their order and their buffers are fixed, only the
        integers that name tokens, positions and slots change.

        While the device runs the step, the host stages the next one for the same
        sequences (their slots' next position reserved, page tables sent, all integers
        but the tokens packed); if the next call brings exactly these sequences, only
        their tokens are filled in before the launch.  Anything else (a sequence ended,
        another joined, a rollback) takes the ordinary way."""
        n = len(entries)
        slots = tuple(e.slot for e in entries)
        ahead, self._ahead = self._ahead, None
        tokens = [int(e.tokens[0]) for e in entries]
        if ahead is not None and ahead.slots == slots and all(self.cache.slots.length(s) == p for s, p in zip(slots, ahead.starts)):
            for t in tokens:
                if not 0 <= t < self.vocab_size:
                    raise ValueError(f"token {t} is outside the vocabulary")
            starts, g, packed = ahead.starts, ahead.graph, ahead.packed
            if not tokens_on_device:
                packed[:n] = tokens
        elif tokens_on_device:
            raise RuntimeError("the staged step does not fit these sequences any more")
        else:
            starts = self.check_entries(entries)
            self.cache.slots.reserve_many([(slot, start + 1, 1) for slot, start in zip(slots, starts)])
            g = self._graph_for(n, max(starts) + 1)
            packed = g.pack(tokens, starts, slots, n)
        count_traffic("h2d", self.cache.sync_tables(), True)
        scores = g.run(packed, keep_tokens=tokens_on_device)[:n]
        self.last_graph = g
        if not borrow_scores:
            scores = scores.clone()
        for slot, start in zip(slots, starts):
            self.cache.slots.commit(slot, start + 1)
        self.steps_run += 1
        # The device is busy now: stage the step after this one.
        try:
            nxt = [start + 1 for start in starts]
            if max(nxt) + 1 <= self.max_seq:
                self.cache.slots.reserve_many([(slot, start + 1, 1) for slot, start in zip(slots, nxt)])
                count_traffic("h2d", self.cache.sync_tables(), True)
                after = self._graph_for(n, max(nxt) + 1)   # another one where the longest sequence crosses a bound
                self._ahead = _Ahead(slots, nxt, after, after.pack(None, nxt, slots, n))
        except CacheError:
            self._ahead = None   # the step itself will say what is wrong, if it comes
        return scores

    def step(self, entries: Sequence[StepEntry], pad_rows_to: int = 1, borrow_scores: bool = False) -> torch.Tensor:
        """Runs the given tokens of every entry as one batch from the cache and returns
        the scores [wanted, vocab] (float32, on the device) at the wanted places, in entry
        order then ``want`` order.  ``pad_rows_to`` adds rows that belong to no sequence;
        they change no result.

        The returned tensor is the caller's own.  With ``borrow_scores`` a decode step may
        instead return a view of the one buffer its captured graph writes: valid until the
        next call of ``step``, which overwrites it in place (the generation loop samples
        from it at once and saves the copy).

        A step that is refused (a bad token, a slot not held or named twice, a wanted index
        outside its tokens, a full cache) raises before anything is reserved or run."""
        if self.use_graphs and pad_rows_to == 1 and entries and all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries) \
                and len({e.slot for e in entries}) == len(entries):
            return self._decode_graph_step(entries, borrow_scores)
        self._ahead, self.last_graph = None, None
        starts = self.check_entries(entries)
        plan = plan_step(entries, starts, pad_rows_to)    # its checks (a slot twice, a wanted index) come before any reservation
        self.cache.slots.reserve_many([(e.slot, start + len(e.tokens), len(e.tokens)) for e, start in zip(entries, starts)])
        count_traffic("h2d", self.cache.sync_tables(), plan.decode)
        v = self._stage(plan)
        ctx = StepContext(
            rows=plan.padded_rows, seqs=plan.seqs, tokens=v["tokens"], row_pos=v["row_pos"], row_slot=v["row_slot"],
            seq_rows=v["seq_rows"], seq_slot=v["seq_slot"], seq_start=v["seq_start"], max_new=plan.max_new,
            max_total=plan.max_total, decode=plan.decode, host_seq_rows=tuple(int(x) for x in plan.seq_rows),
            host_seq_slot=tuple(int(x) for x in plan.seq_slot), host_seq_start=tuple(int(x) for x in plan.seq_start))
        scores = self.model.forward(ctx, self.cache, v["want_rows"], len(plan.want_rows))
        for e, start in zip(entries, starts):
            self.cache.slots.commit(e.slot, start + len(e.tokens))
        self.steps_run += 1
        return scores

    def raise_on_kernel_error(self) -> None:
        """For callers that have just synchronised with the device (read scores or token ids
        back): raises ops.KernelError if a kernel of an earlier step gave up on a bounded
        wait, in which case that step's results are not valid.  Costs a read of host memory."""
        ops.check_status(self.rt.device)

    # ---------------------------------------------------------------------------- accounts
    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for _, part in self.model.named_parts():
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total
