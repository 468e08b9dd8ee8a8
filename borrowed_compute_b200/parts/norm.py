"""RMSNorm: x / sqrt(mean(x^2) + eps) * w, statistics in float32
(crates/bc-infer/src/model.rs:381-389)."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import NORMS, Norm, Runtime, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float):
        super().__init__(size=size, eps=eps)
        self.size, self.eps = int(size), float(eps)

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), role="vector", init="ones")}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, residual: torch.Tensor, out: torch.Tensor, gather: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(residual, self.weight, out, self.eps, gather)
