"""The dense gated feed-forward: down( silu(x gate^T) * (x up^T) ), added into the residual
stream (crates/bc-infer/src/model.rs:341-345).  Gate and up are one product whose epilogue
applies the gate."""

from __future__ import annotations

from typing import Dict

import torch

from . import products
from .base import FEED_FORWARDS, FeedForward, Runtime, StepContext, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)

    def tensors(self) -> Dict[str, TensorSpec]:
        e, f = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": TensorSpec((f, e)),
            "up_proj.weight": TensorSpec((f, e)),
            "down_proj.weight": TensorSpec((e, f)),
        }

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        # Gate rows stacked on up rows: the product's epilogue pairs row j with row F + j.
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        h = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        products.linear(x, self.w_gate_up, h, products.EPI_SWIGLU, "gate/up product")
        products.linear(h, self.w_down, residual, products.EPI_ADD_F32, "down product")
