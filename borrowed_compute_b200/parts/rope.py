"""Rotary position encoding: the table of (cos, sin) a mixer rotates queries and keys with.

Frequencies are theta^(-2i/d), divided per pair by the llama3 long-context factor when the
configuration asks for it (the reference divides by stored factors,
crates/bc-infer/src/model.rs:208-211).  They are computed in float64 and rounded to float32
once.  The angle of (position, pair) is the float32 product of the two, as in the
reference (crates/bc-infer/src/gpu/kernels.h:241); its cosine and sine are taken in float64
and rounded, so the table is as exact as float32 allows at any position.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from ..config.llama import Llama3RopeScaling
from .base import POSITION_ENCODINGS, PositionEncoding, RotaryTable, Runtime

PAIRINGS = {"half": 0, "adjacent": 1}


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[Llama3RopeScaling]) -> torch.Tensor:
    """float32 [head_dim // 2]: radians per position of each rotated pair."""
    out = []
    for i in range(head_dim // 2):
        f = float(theta) ** (-2.0 * i / head_dim)
        if scaling is not None:
            f = scaling.scale_frequency(f)
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def rotary_table(inv_freq: torch.Tensor, positions: int) -> torch.Tensor:
    """float32 [positions, pairs, 2] of (cos, sin) of float32(position) * inv_freq."""
    pos = torch.arange(positions, dtype=torch.float32)
    angle = (pos[:, None] * inv_freq[None, :].to(torch.float32)).to(torch.float64)
    return torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).contiguous()


_tables: Dict[Tuple, RotaryTable] = {}


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, pairing: str = "half", scaling: Optional[Mapping[str, Any]] = None,
                 max_positions: int = 4096):
        super().__init__(head_dim=head_dim, theta=theta, pairing=pairing, scaling=scaling, max_positions=max_positions)
        if pairing not in PAIRINGS:
            raise ValueError(f"rotary pairing {pairing!r} is neither 'half' nor 'adjacent'")
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {head_dim}")
        self.head_dim, self.theta, self.pairing, self.max_positions = int(head_dim), float(theta), pairing, int(max_positions)
        self.scaling = None if scaling is None else Llama3RopeScaling.from_dict(scaling)
        self._table: Optional[RotaryTable] = None

    def load(self, tensors, rt: Runtime) -> None:
        super().load(tensors, rt)
        positions = min(self.max_positions, rt.max_positions) if rt.max_positions else self.max_positions
        key = (self.head_dim, self.theta, self.pairing, self.scaling, positions, str(rt.device))
        if key not in _tables:
            table = rotary_table(inverse_frequencies(self.head_dim, self.theta, self.scaling), positions)
            _tables[key] = RotaryTable(cos_sin=table.to(rt.device), pairing=PAIRINGS[self.pairing])
        self._table = _tables[key]

    def rotary(self) -> Optional[RotaryTable]:
        return self._table


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """A mixer that needs no positions (or learns them elsewhere)."""
