"""A decoder assembled from a ModelSpec: embedding, blocks in scheduled order, final norm,
head.  Nothing here knows an architecture; the sequence of work is the reference's
(crates/bc-infer/src/lib.rs:50-54: embed, forward, logits)."""

from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from ..architectures import resolve
from ..parts import base as P
from ..parts.base import (BLOCKS, EMBEDDINGS, HEADS, NORMS, POSITION_ENCODINGS, CacheNeed, ModelSpec, PartSpec, Runtime, StateNeed,
                          StepContext, TensorSpec)


def _build(registry: P.Registry, spec: PartSpec):
    return registry.get(spec.kind)(**dict(spec.params))


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        for i, run in enumerate(spec.schedule):
            if not 0 <= run.layer < len(spec.layers):
                raise ValueError(f"schedule entry {i} names layer {run.layer}, the model has {len(spec.layers)}")
            if run.memory_of is not None and not (0 <= run.memory_of < i and spec.schedule[run.memory_of].memory_of is None):
                raise ValueError(f"schedule entry {i} reads the memory of entry {run.memory_of}, which is not an earlier owner")
        self.embedding = _build(EMBEDDINGS, spec.embedding)
        self.position = None if spec.position is None else _build(POSITION_ENCODINGS, spec.position)
        self.blocks = [BLOCKS.get(layer.block).build(layer, spec.hidden_size) for layer in spec.layers]
        self.final_norm = _build(NORMS, spec.final_norm)
        self.head = _build(HEADS, spec.head)
        self.rt: Optional[Runtime] = None

    def named_parts(self):
        """(tensor-name prefix, part) of every part of the model; each block lists its own."""
        yield self.spec.embedding.prefix, self.embedding
        if self.position is not None:
            yield self.spec.position.prefix, self.position
        for layer, block in zip(self.spec.layers, self.blocks):
            yield from block.named_parts(layer)
        yield self.spec.final_norm.prefix, self.final_norm
        yield self.spec.head.prefix, self.head

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for prefix, part in self.named_parts():
            for name, spec in part.tensors().items():
                out[prefix + name] = spec
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        for prefix, part in self.named_parts():
            mine = {name: tensors[prefix + name] for name in part.tensors() if prefix + name in tensors}
            part.load(mine, rt)

    def memory_needs(self) -> Tuple[List[Optional[CacheNeed]], List[Optional[StateNeed]], List[Optional[int]]]:
        needs, states, memory_of = [], [], []
        for run in self.spec.schedule:
            mixer = self.blocks[run.layer].memory_part()
            needs.append(None if mixer is None else mixer.cache_need())
            states.append(None if mixer is None else mixer.state_need())
            memory_of.append(run.memory_of)
        return needs, states, memory_of

    def forward(self, ctx: StepContext, cache, want_rows: Optional[torch.Tensor], n_want: int) -> torch.Tensor:
        """Scores [n_want, vocab] float32 at rows ``want_rows`` (all rows if None)."""
        rt = self.rt
        residual = torch.empty((ctx.rows, self.spec.hidden_size), dtype=torch.float32, device=rt.device)
        self.embedding.forward(ctx, residual)
        if self.position is not None:
            self.position.on_embeddings(residual, ctx)
        for i, run in enumerate(self.spec.schedule):
            self.blocks[run.layer].forward(residual, ctx, cache.memory(i), rt)
        h = torch.empty((n_want, self.spec.hidden_size), dtype=rt.dtype, device=rt.device)
        self.final_norm.forward(residual, h, want_rows)
        scores = torch.empty((n_want, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        self.head.forward(h, scores, self.embedding.table())
        return scores


def model_for_config(config: Mapping[str, Any]) -> Tuple[Any, DecoderModel]:
    """The typed configuration and the (unloaded) model a config.json dict describes."""
    arch = resolve(config)
    typed = arch.parse_config(config)
    return typed, DecoderModel(arch.model_spec(typed))


def expected_tensors_for_config(config: Mapping[str, Any]) -> Dict[str, TensorSpec]:
    return model_for_config(config)[1].expected_tensors()
