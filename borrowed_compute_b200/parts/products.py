"""The one place that decides which kernel multiplies matrices.

``linear(x, w, out, epilogue)`` computes ``x @ w.T`` with float accumulation.  On the
32-bit path it is the CUDA-core kernel (tensor cores would round operands to tf32).  For
bfloat16 it is the tcgen05 tensor-core kernel; the CUDA-core kernel on the same operands is
its checked twin and can be forced for a test with ``force_simt``.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops import EPI_ADD_F32, EPI_STORE, EPI_STORE_F32, EPI_SWIGLU  # noqa: F401  (re-exported)

force_simt = False


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, what: str = "") -> None:
    """``what`` names the product for a profile of the step ("qkv", "head", ...)."""
    if ops.timeline is not None and what:
        ops.label = what
        try:
            linear(x, w, out, epilogue)
        finally:
            ops.label = ""
        return
    if x.dtype == torch.bfloat16 and not force_simt and hasattr(ops, "gemm_tc") and ops.gemm_tc_accepts(x, w):
        ops.gemm_tc(x, w, out, epilogue)
    else:
        ops.gemm_simt(x, w, out, epilogue)
