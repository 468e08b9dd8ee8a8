"""Where a step's time goes: every launch of the steps run inside a StepProfile is timed
with CUDA events and summed by class (norm, each product, attention, rotary + append,
embedding, sampling).  The reference times its passes and probes its products the same way,
with its own clock around its own kernels (crates/bc-infer/src/gpu/mod.rs:210-243;
crates/bc-mesh/src/llm.rs:331-339).

Steps inside a profile run launch by launch: the captured decode graph is set aside, and an
event between two launches keeps the second from starting under the first's tail.  The
classes therefore add up to more than a served step takes; their shares, and each class
against its own bytes or operations, are what to read.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from .engine import Engine


class StepProfile:
    """``with StepProfile(engine) as p: engine.step(...)``, then ``p.classes()``."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.records: List[tuple] = []
        self._graphs = engine.use_graphs

    def __enter__(self) -> "StepProfile":
        if ops.timeline is not None:
            raise RuntimeError("a step profile is already being taken")
        self._graphs = self.engine.use_graphs
        self.engine.use_graphs = False
        ops.timeline = self.records
        return self

    def __exit__(self, *exc) -> None:
        ops.timeline = None
        self.engine.use_graphs = self._graphs

    def classes(self, steps: int = 1) -> Dict[str, Dict[str, float]]:
        """class -> {"us": microseconds a step, "launches": launches a step}, over the
        ``steps`` steps that ran inside the profile."""
        torch.cuda.synchronize(self.engine.rt.device)
        out: Dict[str, Dict[str, float]] = {}
        for cls, _, start, end in self.records:
            entry = out.setdefault(cls, {"us": 0.0, "launches": 0.0})
            entry["us"] += start.elapsed_time(end) * 1000.0 / steps
            entry["launches"] += 1.0 / steps
        return out
