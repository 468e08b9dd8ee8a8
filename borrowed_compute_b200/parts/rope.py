"""Rotary position encoding: the table of (cos, sin) a mixer rotates queries and keys with.

Frequencies are theta^(-2i/d), divided per pair by the llama3 long-context factor when the
configuration asks for it (the reference divides by stored factors,
crates/bc-infer/src/model.rs:208-211).  They are computed in float64 and rounded to float32
once.  The angle of (position, pair) is the float32 product of the two, as in the
reference (crates/bc-infer/src/gpu/kernels.h:241); its cosine and sine are taken in float64
and rounded, so the table is as exact as float32 allows at any position.
"""

from __future__ import annotations

import math
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from .base import POSITION_ENCODINGS, PositionEncoding, RotaryTable, Runtime

PAIRINGS = {"half": 0, "adjacent": 1}


def llama3_scaled_frequency(f: float, factor: float, low_freq_factor: float, high_freq_factor: float, original_max_positions: int) -> float:
    """The llama3 rule for long contexts, for one frequency ``f`` (radians a position):
    wavelengths shorter than original / high_freq_factor keep their frequency, those longer
    than original / low_freq_factor are slowed by ``factor``, and those between blend the
    two linearly in original / wavelength.  The reference only divides each frequency by a
    stored per-pair factor (crates/bc-infer/src/model.rs:208-211); this rule is what
    produces those factors."""
    wavelen = 2.0 * math.pi / f
    orig = float(original_max_positions)
    if wavelen < orig / high_freq_factor:
        return f
    if wavelen > orig / low_freq_factor:
        return f / factor
    t = (orig / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    return (1.0 - t) * f / factor + t * f


def _llama3_rule(d: Mapping[str, Any]) -> Callable[[float], float]:
    try:
        factor, low, high = float(d["factor"]), float(d["low_freq_factor"]), float(d["high_freq_factor"])
        orig = int(d["original_max_position_embeddings"])
    except (KeyError, TypeError, ValueError) as e:
        raise ValueError(f"llama3 frequency scaling needs factor, low_freq_factor, high_freq_factor and "
                         f"original_max_position_embeddings as numbers, got {dict(d)!r}") from e
    if factor <= 0 or high <= low or orig <= 0:
        raise ValueError(f"llama3 frequency scaling values are inconsistent: {dict(d)!r}")
    return lambda f: llama3_scaled_frequency(f, factor, low, high, orig)


# Rules that rescale rotary frequencies, by the name a configuration gives them.  Each takes
# the rule's own numbers (a plain mapping) and returns frequency -> frequency.
FREQUENCY_SCALINGS: Dict[str, Callable[[Mapping[str, Any]], Callable[[float], float]]] = {"llama3": _llama3_rule}


def frequency_rule(scaling: Optional[Mapping[str, Any]]) -> Optional[Callable[[float], float]]:
    if scaling is None:
        return None
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind not in FREQUENCY_SCALINGS:
        raise ValueError(f"rotary frequency scaling {kind!r} is not known (known: {sorted(FREQUENCY_SCALINGS)})")
    return FREQUENCY_SCALINGS[kind](scaling)


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[Mapping[str, Any]]) -> torch.Tensor:
    """float32 [head_dim // 2]: radians per position of each rotated pair; ``scaling`` is
    a mapping {"rope_type": name, ...the rule's numbers} or None."""
    rule = frequency_rule(scaling)
    out = []
    for i in range(head_dim // 2):
        f = float(theta) ** (-2.0 * i / head_dim)
        out.append(f if rule is None else rule(f))
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
        self.scaling = None if scaling is None else dict(scaling)
        frequency_rule(self.scaling)   # refuses an unknown or inconsistent rule when the part is built
        self._table: Optional[RotaryTable] = None

    def load(self, tensors, rt: Runtime) -> None:
        super().load(tensors, rt)
        positions = min(self.max_positions, rt.max_positions) if rt.max_positions else self.max_positions
        key = (self.head_dim, self.theta, self.pairing, None if self.scaling is None else tuple(sorted(self.scaling.items())),
               positions, str(rt.device))
        if key not in _tables:
            table = rotary_table(inverse_frequencies(self.head_dim, self.theta, self.scaling), positions)
            _tables[key] = RotaryTable(cos_sin=table.to(rt.device), pairing=PAIRINGS[self.pairing])
        self._table = _tables[key]

    def rotary(self) -> Optional[RotaryTable]:
        return self._table


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """A mixer that needs no positions (or learns them elsewhere)."""
