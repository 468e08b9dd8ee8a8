"""Errors of the kernels that reach the caller: a bounded wait that runs out (made to, the
harmless way: a launch that expects bytes nobody sends, with the wait limit set to about a
millisecond) ends its launch, frees what it holds, and is reported on the host; the launch
after it is right.  And the start-up check of every product against float64 sums."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import TINY_A, seeded_tokens

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def operands():
    r = np.random.default_rng(0)
    x = torch.from_numpy(r.standard_normal((8, 512)).astype(np.float32)).cuda().bfloat16()
    w = torch.from_numpy(r.standard_normal((300, 512)).astype(np.float32) * 0.1).cuda().bfloat16()
    return x, w, x.float().cpu().numpy().astype(np.float64) @ w.float().cpu().numpy().astype(np.float64).T


def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_right():
    from borrowed_compute_b200 import ops

    ops.bind_status()
    torch.cuda.synchronize()
    ops.check_status()
    x, w, want = operands()
    out = torch.full((8, 300), 7.0, dtype=torch.float32, device="cuda")
    ops.set_wait_cycles(2_000_000)                      # about a millisecond
    try:
        ops.gemm_tc_test_starve_next_launch()
        ops.gemm_tc(x, w, out, ops.EPI_STORE_F32, splits=1)
        torch.cuda.synchronize()                        # the launch ended by itself: its waits gave up, its blocks tore down
        with pytest.raises(ops.KernelError, match="tensor-core product.*ran out") as err:
            ops.check_status()
        # the loader, the MMA thread and the epilogue all wait on what the missing bytes hold up; whichever limit ends first is named
        assert any(f"code {c}" in str(err.value) for c in (1, 2, 3))
        assert bool((out == 7.0).all()), "a block that gave up writes nothing"
        ops.check_status()                              # reported once, then clear on both sides
        assert ops.gemm_tc_status() == 0
    finally:
        ops.set_wait_cycles(0)
    # The launches after it find the SMs' tensor memory free and give the right product, split or not.
    for splits in (1, 4):
        ops.gemm_tc(x, w, out, ops.EPI_STORE_F32, splits=splits)
        torch.cuda.synchronize()
        assert np.abs(out.cpu().numpy() - want).max() <= 1e-3 * (1 + np.abs(want).max())
    ops.check_status()


def test_the_entry_point_raises_when_a_kernel_gave_up(model_folders):
    from borrowed_compute_b200 import Local, ops

    folder, cfg, weights = model_folders("A", "bfloat16")
    model = Local.load(folder, dtype="bfloat16", max_tokens=256)
    tokens = seeded_tokens(1, 9, cfg["vocab_size"])
    good = model.scores(tokens, 0)
    model.reset()
    ops.set_wait_cycles(2_000_000)
    try:
        ops.gemm_tc_test_starve_next_launch()           # the step's first product never gets its operands
        with pytest.raises(ops.KernelError, match="ran out"):
            model.scores(tokens, 0)
    finally:
        ops.set_wait_cycles(0)
    model.reset()
    assert torch.equal(model.scores(tokens, 0), good), "the engine is whole again after the report"
    out, _ = model.generate([tokens], 4)
    assert len(out[0]) == 4


def test_the_start_up_check_passes_and_catches_a_wrong_product(monkeypatch):
    from borrowed_compute_b200 import ops

    dev = torch.device("cuda:0")
    ops._self_checked.discard(0)
    ops.self_check(dev)
    assert 0 in ops._self_checked
    real = ops.gemm_tc

    def off_by_a_row(x, w, out, epilogue, splits=None):
        real(x, w, out, epilogue, splits)
        if epilogue == ops.EPI_ADD_F32:
            out[-1, 5] += 0.5

    ops._self_checked.discard(0)
    monkeypatch.setattr(ops, "gemm_tc", off_by_a_row)
    with pytest.raises(ops.KernelError, match="self-check.*add_f32"):
        ops.self_check(dev)
    monkeypatch.undo()
    ops.self_check(dev)
