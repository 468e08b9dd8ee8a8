"""Token embedding and the output head (crates/bc-infer/src/model.rs:270-280, 361-370)."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from . import products
from .base import EMBEDDINGS, HEADS, Embedding, Head, Runtime, StepContext, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, hidden_size: int):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.weight = tensors["weight"].contiguous()

    def forward(self, ctx: StepContext, residual: torch.Tensor) -> None:
        ops.embed(self.weight, ctx.tokens[: residual.shape[0]], residual)

    def table(self) -> Optional[torch.Tensor]:
        return self.weight


@HEADS.register("linear_head")
class LinearHead(Head):
    """Scores = x W^T in float32.  A tied head has no tensor of its own and multiplies by
    the embedding table (model.rs:200); a folder that still stores one is tolerated."""

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool = False):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, tied=tied)
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.weight = None if self.tied else tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, tied: Optional[torch.Tensor]) -> None:
        w = tied if self.tied else self.weight
        if w is None:
            raise RuntimeError("a tied head needs the embedding's table")
        products.linear(x, w, out, products.EPI_STORE_F32, "head product")
