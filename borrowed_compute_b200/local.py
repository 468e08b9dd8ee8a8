"""The Python entry point, in the reference's manner.

The reference's library face is ``Local::load(source)`` / ``Local::scores(tokens, pos)``
(crates/bc-infer/src/lib.rs:26-55) and ``Llm::generate(prompt, max_tokens, Sampling,
on_text) -> (tokens, Stats)`` (crates/bc-mesh/src/llm.rs:511).  The same names and meanings
are kept; prompts are token ids (text and tokenizers are outside this library), and
``generate`` takes several prompts at once.
"""

from __future__ import annotations

from typing import Any, Callable, List, Mapping, Optional, Sequence, Tuple, Union

import torch

from .engine import Engine, EngineBackend, Stats, StepEntry, run_generation
from .sampling import Sampling


class Local:
    """A whole model on this device."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self._slot: Optional[int] = None

    @classmethod
    def load(cls, source: str, dtype: str = "bfloat16", device: str = "cuda:0", max_tokens: Optional[int] = None,
             max_slots: Optional[int] = None, max_seq: Optional[int] = None,
             progress: Optional[Callable[[int, int], None]] = None) -> "Local":
        """Loads a model folder (config.json + safetensors); ``progress(done, total)`` reports
        the tensors brought to the device as it goes (lib.rs:33-47, ``load_with``)."""
        return cls(Engine.from_folder(source, dtype=dtype, device=device, max_tokens=max_tokens, max_slots=max_slots, max_seq=max_seq,
                                      progress=progress))

    @classmethod
    def random(cls, config: Mapping[str, Any], seed: int = 0, dtype: str = "bfloat16", device: str = "cuda:0",
               max_tokens: Optional[int] = None, max_slots: Optional[int] = None, max_seq: Optional[int] = None) -> "Local":
        """A model of random weights for a configuration, without a folder."""
        return cls(Engine.from_random(config, seed, dtype=dtype, device=device, max_tokens=max_tokens, max_slots=max_slots, max_seq=max_seq))

    @property
    def stop_ids(self) -> Tuple[int, ...]:
        return tuple(self.engine.stop_ids)

    def scores(self, tokens: Sequence[int], pos: int) -> torch.Tensor:
        """Scores after each of ``tokens``, placed at ``pos..`` of this object's own
        conversation (rows x vocab, float32, on the host).  ``pos`` below the cached length
        drops what lay after it; ``pos`` past it is an error (lib.rs:50-54; model.rs:303-305)."""
        if self._slot is None:
            self._slot = self.engine.acquire()
        have = self.engine.length(self._slot)
        if pos > have:
            raise ValueError(f"position {pos} skips past the {have} cached tokens")
        if pos < have:
            self.engine.rollback(self._slot, pos)
        out = self.engine.step([StepEntry(self._slot, list(tokens), want=tuple(range(len(tokens))))]).cpu()
        self.engine.raise_on_kernel_error()
        return out

    def reset(self) -> None:
        if self._slot is not None:
            self.engine.release(self._slot)
            self._slot = None

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], max_tokens: int,
                 sampling: Union[Sampling, Sequence[Sampling], None] = None,
                 on_token: Optional[Callable[[int, int], None]] = None, stop_ids: Optional[Sequence[int]] = None,
                 max_batch: Optional[int] = None, include_stop: bool = False) -> Tuple[Any, Stats]:
        """Generates up to ``max_tokens`` after each prompt.  One prompt (a list of ids)
        gives one list back, several give a list of lists.  ``stop_ids`` default to the
        model's end-of-sequence ids (config.json's and generation_config.json's); a stop id
        ends a sequence and is not returned, unless ``include_stop`` asks for it as the
        sequence's last id (the reference's self-fed runs return it so,
        crates/bc-mesh/src/engine.rs:355)."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        batch: List[Sequence[int]] = [prompts] if single else list(prompts)
        if sampling is None:
            sampling = Sampling()
        samplings = [sampling] * len(batch) if isinstance(sampling, Sampling) else list(sampling)
        backend = EngineBackend(self.engine, max_batch=max_batch)
        out, stats = run_generation(backend, batch, max_tokens, samplings, self.stop_ids if stop_ids is None else stop_ids, on_token,
                                    include_stop=include_stop)
        return (out[0] if single else out), stats
