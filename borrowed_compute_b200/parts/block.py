"""The pre-norm residual block: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(crates/bc-infer/src/model.rs:323-345)."""

from __future__ import annotations

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, RunMemory, Runtime, StepContext


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    ROLES = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        h = torch.empty((residual.shape[0], self.hidden_size), dtype=rt.dtype, device=residual.device)
        self.norm1.forward(residual, h)
        self.mixer.forward(h, residual, ctx, mem)
        self.norm2.forward(residual, h)
        self.feed_forward.forward(h, residual, ctx)
