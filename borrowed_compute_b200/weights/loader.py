"""From a model folder to tensors on the device, by tensor name.

The reference looks tensors up by name in a map and fails on the first missing one
(crates/bc-infer/src/model.rs:176-204).  Here everything a model declares is checked
against everything the folder holds first, and one error lists every missing tensor, every
unexpected one and every wrong shape.
"""

from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping, Tuple

import torch

from ..config.errors import ConfigError, WeightsError
from ..parts.base import Runtime, TensorSpec
from .safetensors_io import TensorSource

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            cfg = json.load(f)
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not JSON: {e}") from e
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path} does not hold an object")
    return cfg


def read_generation_stop_ids(folder: str, vocab_size: int) -> tuple:
    """The end-of-sequence ids of ``generation_config.json``, if the folder has one: an
    integer or a list of them.  Published folders name there the ids that end a reply
    (several, for chat models), beside the one of config.json."""
    path = os.path.join(folder, "generation_config.json")
    if not os.path.isfile(path):
        return ()
    try:
        with open(path) as f:
            eos = json.load(f).get("eos_token_id")
    except (OSError, json.JSONDecodeError, AttributeError) as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    if eos is None:
        return ()
    ids = [eos] if isinstance(eos, int) and not isinstance(eos, bool) else eos
    if not isinstance(ids, (list, tuple)) or not all(isinstance(e, int) and not isinstance(e, bool) for e in ids):
        raise ConfigError(f"{path}: 'eos_token_id' must be an integer or a list of integers, got {eos!r}")
    for e in ids:
        if not 0 <= e < vocab_size:
            raise ConfigError(f"{path}: eos_token_id {e} is outside the vocabulary of {vocab_size}")
    return tuple(ids)


def check_tensors(expected: Mapping[str, TensorSpec], have: Mapping[str, Tuple[torch.dtype, Tuple[int, ...]]], where: str) -> None:
    """Raises one WeightsError naming all that is missing, unexpected or misshapen."""
    missing = [n for n, s in expected.items() if n not in have and not s.optional]
    unexpected = [n for n in have if n not in expected]
    wrong = []
    for n, s in expected.items():
        if n in have:
            dtype, shape = have[n]
            if tuple(shape) != tuple(s.shape):
                wrong.append(f"{n}: expected {list(s.shape)}, found {list(shape)}")
            elif (s.role == "index" and dtype not in _INTS) or (s.role != "index" and dtype not in _FLOATS):
                wrong.append(f"{n}: stored as {dtype}, which a tensor of role '{s.role}' cannot be")
    if missing or unexpected or wrong:
        parts = [f"the tensors in {where} do not fit the model:"]
        if missing:
            parts.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            parts.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            parts.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightsError("\n".join(parts))


def device_type(spec: TensorSpec, stored: torch.dtype, rt: Runtime) -> torch.dtype:
    """The type a tensor takes on the device (see TensorSpec.role)."""
    if spec.role == "index":
        return torch.int32
    if spec.role == "vector":
        return torch.float32
    return rt.dtype


def load_tensors(expected: Mapping[str, TensorSpec], source: TensorSource, rt: Runtime,
                 progress: Callable[[int, int], None] | None = None) -> Dict[str, torch.Tensor]:
    """Checks the folder against ``expected`` and brings every expected tensor to the
    device in the type its role asks for."""
    have = {n: source.info(n) for n in source.names()}
    check_tensors(expected, have, source.folder)
    out: Dict[str, torch.Tensor] = {}
    total = sum(1 for n in expected if n in have)
    for i, (name, spec) in enumerate(expected.items()):
        if name not in have:
            continue
        t = source.tensor(name)
        out[name] = t.to(device=rt.device, dtype=device_type(spec, t.dtype, rt)).contiguous()
        if progress is not None:
            progress(i + 1, total)
    return out
