"""Random weights from a configuration and a seed, and the model folder that holds them.

Every tensor is drawn on its own from a generator seeded by (seed, tensor name), so a
tensor's values do not depend on which other tensors exist: normal(0, 0.02) for matrices,
ones for norm weights.  The reference's counterpart is its test fixture
(crates/bc-infer/src/fixtures.rs:7-60).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping

import torch

from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors

STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype, device: torch.device | str = "cpu") -> torch.Tensor:
    """One tensor's values.  Drawn in float32 and then rounded to ``dtype``; on a CUDA
    device the draw uses that device's generator (other values than the CPU's)."""
    if spec.role == "index":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    t.normal_(0.0, STD, generator=gen)
    return t.to(dtype)


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype, device: torch.device | str = "cpu") -> Dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, dtype, device) for name, spec in expected.items() if not spec.optional}


def write_model_folder(folder: str, config: Mapping[str, Any], seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for random weights of the
    architecture that ``config`` names, and returns the folder."""
    from ..engine.model import expected_tensors_for_config

    expected = expected_tensors_for_config(config)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(config), f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_tensors(expected, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
