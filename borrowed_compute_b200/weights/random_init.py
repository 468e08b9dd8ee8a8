"""Random weights from a configuration and a seed, and the model folder that holds them.

Every value is a pure function of (seed, tensor name, element index): normal(0, 0.02) for
matrices, ones for norm weights.  A tensor's values therefore do not depend on which other
tensors exist, on the device, or on how the work is cut, and the host (NumPy, here) and
the device (csrc/random_init.cu) produce the same bits: a model drawn on the device for a
benchmark can be drawn again on the host for a check.  The reference's counterpart is its
test fixture, deterministic everywhere (crates/bc-infer/src/fixtures.rs:7-60).

The draw: a 64-bit key from the seed and the name; splitmix64 of key + (index + 1) * golden
ratio gives two 24-bit uniforms; Box and Muller's transform turns them into one normal
deviate.  Its logarithm, sine and cosine are short polynomials evaluated with single
float32 additions, multiplications, one division and one square root, all of which IEEE 754
rounds correctly, so both implementations agree to the bit.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping

import numpy as np
import torch

from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors

STD = 0.02
_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


def _mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's stream: FNV-1a of the name, mixed with the seed."""
    h = 0xCBF29CE484222325
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _MASK
    return _mix64((int(seed) & _MASK) ^ h)


def _f(x: float) -> np.float32:
    return np.float32(x)


def normal_deviates(key: int, count: int, first: int = 0) -> np.ndarray:
    """float32 [count]: the standard normal deviates of elements first .. first + count of
    the stream ``key``; the NumPy mirror of normal_deviate() in csrc/random_init.cu, step
    for step."""
    with np.errstate(over="ignore"):
        idx = np.arange(first + 1, first + count + 1, dtype=np.uint64)
        z = np.uint64(key) + idx * np.uint64(_GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        h = z ^ (z >> np.uint64(31))
    a = (h >> np.uint64(40)).astype(np.uint32)
    b = ((h >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.uint32)
    u = (a + np.uint32(1)).astype(np.float32) * _f(5.9604644775390625e-08)
    m, e = np.frexp(u)
    low = m < _f(0.70710678118654752)
    m = np.where(low, m * _f(2.0), m).astype(np.float32)
    e = np.where(low, e - 1, e).astype(np.int32)
    s = (m + _f(-1.0)) / (m + _f(1.0))
    s2 = s * s
    p = np.full_like(s, _f(0.090909090909090909))
    for c in (0.11111111111111111, 0.14285714285714285, 0.2, 0.33333333333333333):
        p = _f(c) + s2 * p
    ln_m = _f(2.0) * (s + s * (s2 * p))
    ln_u = e.astype(np.float32) * _f(0.69314718055994531) + ln_m
    radius = np.sqrt(_f(-2.0) * ln_u)
    quadrant = b >> np.uint32(22)
    x = ((b & np.uint32(0x3FFFFF)).astype(np.float32) * _f(2.384185791015625e-07)) * _f(1.5707963267948966)
    x2 = x * x
    sn = np.full_like(x, _f(1.6059043836821613e-10))
    for c in (-2.5052108385441719e-08, 2.7557319223985891e-06, -1.9841269841269841e-04, 8.3333333333333333e-03,
              -1.6666666666666667e-01):
        sn = _f(c) + x2 * sn
    sn = x + x * (x2 * sn)
    cs = np.full_like(x, _f(-1.1470745597729725e-11))
    for c in (2.0876756987868099e-09, -2.7557319223985888e-07, 2.4801587301587302e-05, -1.3888888888888889e-03,
              4.1666666666666664e-02, -0.5, 1.0):
        cs = _f(c) + x2 * cs
    c = np.where(quadrant == 0, cs, np.where(quadrant == 1, -sn, np.where(quadrant == 2, -cs, sn)))
    out = radius * c
    assert out.dtype == np.float32
    return out


def _normal_on_host(shape, key: int, dtype: torch.dtype) -> torch.Tensor:
    count = 1
    for s in shape:
        count *= int(s)
    out = np.empty(count, dtype=np.float32)
    for first in range(0, count, 1 << 22):          # in pieces, to bound the temporaries
        n = min(1 << 22, count - first)
        out[first:first + n] = normal_deviates(key, n, first) * _f(STD)
    return torch.from_numpy(out).reshape(tuple(shape)).to(dtype)


def _normal_on_device(shape, key: int, dtype: torch.dtype, device) -> torch.Tensor:
    from .. import ops

    out = torch.empty(tuple(shape), dtype=dtype, device=device)
    ops.random_normal(out, key, STD)
    return out


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype, device: torch.device | str = "cpu") -> torch.Tensor:
    """One tensor's values: drawn in float32, then rounded to ``dtype``; the same bits
    whether ``device`` is the host or a CUDA device."""
    if spec.role == "index":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    key = tensor_key(seed, name)
    if torch.device(device).type == "cuda":
        return _normal_on_device(spec.shape, key, dtype, device)
    return _normal_on_host(spec.shape, key, dtype)


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
