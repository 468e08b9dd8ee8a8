"""The tcgen05 product against a float64 product of the same bf16 operands, at shapes that
exercise every token tile, ragged edges in all three dimensions, split-K, and all epilogues."""

from __future__ import annotations

import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

SHAPES = [
    # T, N, K, splits
    (1, 128, 64, 1), (16, 128, 128, 1), (5, 70, 176, 1), (37, 320, 96, 1), (64, 256, 256, 1), (100, 200, 128, 1),
    (300, 130, 192, 1), (8, 512, 4096, 4), (33, 256, 2048, 3), (3, 100, 1024, 2), (600, 384, 512, 1),
]


def operands(T, N, K, seed):
    r = np.random.default_rng(seed)
    x = torch.from_numpy(r.standard_normal((T, K)).astype(np.float32)).cuda().to(torch.bfloat16)
    w = torch.from_numpy((r.standard_normal((2 * N, K)) / math.sqrt(K)).astype(np.float32)).cuda().to(torch.bfloat16)
    return x, w


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("T,N,K,splits", SHAPES)
def test_gemm_tc_all_epilogues(T, N, K, splits):
    from borrowed_compute_b200 import ops

    x, w = operands(T, N, K, T * 1000 + N)
    full = f64(x) @ f64(w).T
    scale = 1.0 + np.abs(full).max()
    wn = w[:N].contiguous()
    out32 = torch.full((T, N), 7.0, dtype=torch.float32, device="cuda")
    ops.gemm_tc(x, wn, out32, ops.EPI_STORE_F32, splits=splits)
    assert ops.gemm_tc_status() == 0
    assert np.abs(f64(out32) - full[:, :N]).max() <= 2e-5 * scale, "float store"
    again = torch.empty_like(out32)
    ops.gemm_tc(x, wn, again, ops.EPI_STORE_F32, splits=splits)
    assert torch.equal(out32, again), "the same launch twice must give the same bits"
    out16 = torch.empty((T, N), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc(x, wn, out16, ops.EPI_STORE, splits=splits)
    assert np.abs(f64(out16) - full[:, :N]).max() <= 2.0 ** -8 * scale, "bf16 store"
    base = torch.from_numpy(np.random.default_rng(1).standard_normal((T, N)).astype(np.float32)).cuda()
    acc = base.clone()
    ops.gemm_tc(x, wn, acc, ops.EPI_ADD_F32, splits=splits)
    assert np.abs(f64(acc) - (f64(base) + full[:, :N])).max() <= 2e-5 * scale, "residual add"
    g, u = full[:, :N], full[:, N:]
    ref = g / (1 + np.exp(-g)) * u
    ops.gemm_tc(x, w, out16, ops.EPI_SWIGLU, splits=splits)
    assert np.abs(f64(out16) - ref).max() <= 2.0 ** -8 * (1 + np.abs(ref).max()), "SwiGLU"
    unsplit = torch.empty_like(out16)
    ops.gemm_tc(x, w, unsplit, ops.EPI_SWIGLU, splits=1)
    assert np.abs(f64(unsplit) - ref).max() <= 2.0 ** -8 * (1 + np.abs(ref).max()), "SwiGLU, one split"
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("T,N,K,splits", [(8, 512, 4096, 4), (33, 256, 2048, 3), (3, 100, 1024, 2), (8, 384, 2048, 8), (61, 130, 1536, 5), (8, 256, 4096, 12)])
def test_gemm_tc_splits_agree_through_cluster_and_through_scratch(T, N, K, splits):
    """Splits that add up inside a thread-block cluster give the bits of splits that add up
    through scratch memory (the same order of additions), for every epilogue."""
    from borrowed_compute_b200 import ops

    x, w = operands(T, N, K, T + N + K)
    wn = w[:N].contiguous()
    base = torch.from_numpy(np.random.default_rng(2).standard_normal((T, N)).astype(np.float32)).cuda()
    results = []
    try:
        for clustered in (True, False):
            ops.set_gemm_tc_cluster(clustered)
            out32 = torch.full((T, N), 7.0, dtype=torch.float32, device="cuda")
            ops.gemm_tc(x, wn, out32, ops.EPI_STORE_F32, splits=splits)
            out16 = torch.full((T, N), 7.0, dtype=torch.bfloat16, device="cuda")
            ops.gemm_tc(x, wn, out16, ops.EPI_STORE, splits=splits)
            acc = base.clone()
            ops.gemm_tc(x, wn, acc, ops.EPI_ADD_F32, splits=splits)
            act = torch.full((T, N), 7.0, dtype=torch.bfloat16, device="cuda")
            ops.gemm_tc(x, w, act, ops.EPI_SWIGLU, splits=splits)
            results.append((out32, out16, acc, act))
    finally:
        ops.set_gemm_tc_cluster(True)
    assert ops.gemm_tc_status() == 0
    for a, b, name in zip(results[0], results[1], ("float store", "bf16 store", "residual add", "SwiGLU")):
        assert torch.equal(a, b), name
    full = f64(x) @ f64(wn).T
    assert np.abs(f64(results[0][0]) - full).max() <= 2e-5 * (1.0 + np.abs(full).max())


@pytest.mark.parametrize("T,N,K", [(300, 130, 192), (600, 384, 512), (129, 128, 64), (1000, 1030, 448), (513, 700, 72), (2048, 512, 1024)])
@pytest.mark.parametrize("paired", [True, False, 64, 128, 192])
def test_gemm_tc_many_tokens_on_pairs_of_sms_and_on_single_blocks(T, N, K, paired):
    """More than 128 tokens: the tile shared by two SMs (cta_group::2) and the tile of one
    block, every epilogue, edges in all three dimensions, against the float64 product."""
    from borrowed_compute_b200 import ops

    x, w = operands(T, N, K, T + 3 * N + K)
    full = f64(x) @ f64(w).T
    scale = 1.0 + np.abs(full).max()
    wn = w[:N].contiguous()
    base = torch.from_numpy(np.random.default_rng(3).standard_normal((T, N)).astype(np.float32)).cuda()
    try:
        ops.set_gemm_tc_pair(bool(paired))
        ops.set_gemm_tc_pair_tokens(0 if isinstance(paired, bool) else paired)   # a number: that many tokens a paired tile
        out32 = torch.full((T, N), 7.0, dtype=torch.float32, device="cuda")
        ops.gemm_tc(x, wn, out32, ops.EPI_STORE_F32, splits=1)
        out16 = torch.full((T, N), 7.0, dtype=torch.bfloat16, device="cuda")
        ops.gemm_tc(x, wn, out16, ops.EPI_STORE, splits=1)
        acc = base.clone()
        ops.gemm_tc(x, wn, acc, ops.EPI_ADD_F32, splits=1)
        act = torch.full((T, N), 7.0, dtype=torch.bfloat16, device="cuda")
        ops.gemm_tc(x, w, act, ops.EPI_SWIGLU, splits=1)
    finally:
        ops.set_gemm_tc_pair(True)
        ops.set_gemm_tc_pair_tokens(0)
    assert ops.gemm_tc_status() == 0
    assert np.abs(f64(out32) - full[:, :N]).max() <= 2e-5 * scale, "float store"
    assert np.abs(f64(out16) - full[:, :N]).max() <= 2.0 ** -8 * scale, "bf16 store"
    assert np.abs(f64(acc) - (f64(base) + full[:, :N])).max() <= 2e-5 * scale, "residual add"
    g, u = full[:, :N], full[:, N:]
    ref = g / (1 + np.exp(-g)) * u
    assert np.abs(f64(act) - ref).max() <= 2.0 ** -8 * (1 + np.abs(ref).max()), "SwiGLU"


def test_gemm_tc_matches_the_cuda_core_twin():
    from borrowed_compute_b200 import ops

    x, w = operands(50, 300, 640, 3)
    a = torch.empty((50, 300), dtype=torch.float32, device="cuda")
    b = torch.empty_like(a)
    ops.gemm_tc(x, w[:300].contiguous(), a, ops.EPI_STORE_F32)
    ops.gemm_simt(x, w[:300].contiguous(), b, ops.EPI_STORE_F32)
    assert (a - b).abs().max().item() <= 1e-5 * (1 + b.abs().max().item())


def test_gemm_tc_refuses_what_it_cannot_do():
    from borrowed_compute_b200 import ops

    x, w = operands(4, 64, 100, 4)   # K = 100 is no multiple of 8
    assert not ops.gemm_tc_accepts(x, w)
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.gemm_tc(x, w[:64].contiguous(), torch.empty((4, 64), dtype=torch.float32, device="cuda"), ops.EPI_STORE_F32)
