from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registers the built-in parts)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheNeed, Embedding,
                   FeedForward, Head, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, Registry, RotaryTable,
                   RunMemory, RunSpec, Runtime, StateNeed, StepContext, TensorSpec)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheNeed", "Embedding",
    "FeedForward", "Head", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec", "PositionEncoding", "Registry",
    "RotaryTable", "RunMemory", "RunSpec", "Runtime", "StateNeed", "StepContext", "TensorSpec",
]
