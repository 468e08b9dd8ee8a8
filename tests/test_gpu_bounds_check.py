"""The bounds-checked mode of the launchers: indices that would reach past what they index
are named and refused on the host before anything is launched, and a whole engine runs in
that mode with the results it has without it."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import seeded_tokens, tolerance

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture
def checked():
    from borrowed_compute_b200 import ops

    was = ops.bounds_check
    ops.bounds_check = True
    yield ops
    ops.bounds_check = was


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device="cuda")


def test_bad_indices_are_named_and_nothing_is_launched(checked):
    ops = checked
    table = torch.zeros((10, 16), dtype=torch.bfloat16, device="cuda")
    out = torch.full((3, 16), 7.0, dtype=torch.float32, device="cuda")
    before = ops.launches
    with pytest.raises(ops.KernelError, match=r"embed: tokens\[1\] = 10 is outside \[0, 10\)"):
        ops.embed(table, i32([3, 10, 0]), out)
    assert ops.launches == before and bool((out == 7.0).all())
    x = torch.randn(4, 16, device="cuda")
    with pytest.raises(ops.KernelError, match=r"rmsnorm: gather\[0\] = 4"):
        ops.rmsnorm(x, torch.ones(16, device="cuda"), torch.empty((1, 16), device="cuda"), 1e-5, i32([4]))
    H, G, D, n_pages = 2, 1, 16, 4
    k = torch.zeros((n_pages, G, 64, D), dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    q = torch.zeros((2, H * D), dtype=torch.bfloat16, device="cuda")
    o = torch.empty_like(q)
    pages = i32([[0, 1], [2, -1]])
    ops.attention_decode(q, H * D, k, v, pages, i32([100, 5]), i32([0, 1]), o, H, G, D)            # all in range
    with pytest.raises(ops.KernelError, match=r"row_slot\[1\] = 2 is outside \[-1, 2\)"):
        ops.attention_decode(q, H * D, k, v, pages, i32([100, 5]), i32([0, 2]), o, H, G, D)
    with pytest.raises(ops.KernelError, match=r"row_pos\[0\] = 128 is outside \[0, 128\)"):
        ops.attention_rows(q, H * D, k, v, pages, i32([128, 5]), i32([0, 1]), o, H, G, D)
    with pytest.raises(ops.KernelError, match=r"page_table\[1\] = 4 is outside \[-1, 4\)"):
        ops.attention_decode(q, H * D, k, v, i32([[0, 4], [2, -1]]), i32([100, 5]), i32([0, 1]), o, H, G, D)
    ops.attention_decode(q, H * D, k, v, pages, i32([100, 500]), i32([0, -1]), o, H, G, D)           # a padding row's position is nobody's
    qkv = torch.zeros((2, (H + 2 * G) * D), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match=r"a sequence's last position \+ 1\[0\] = 131"):
        ops.attention_prefill(qkv, (H + 2 * G) * D, k, v, pages, i32([0, 2]), i32([0]), i32([129]), o, 1, 2, H, G, D)


def test_an_engine_runs_in_the_checked_mode(checked, model_folders):
    import plain_llama
    from borrowed_compute_b200 import Engine, StepEntry

    folder, cfg, weights = model_folders("B", "bfloat16")
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=512)
    assert not eng.use_graphs, "every step is checked: none is replayed from a graph"
    tokens = seeded_tokens(4, 80, cfg["vocab_size"])
    ref = plain_llama.logits(cfg, weights, tokens)
    s = eng.acquire()
    got = [eng.step([StepEntry(s, tokens[:70], want=tuple(range(70)))]).cpu().numpy()]
    got += [eng.step([StepEntry(s, [t], want=(0,))]).cpu().numpy() for t in tokens[70:]]
    eng.release(s)
    assert np.abs(np.concatenate(got) - ref).max() <= tolerance("bfloat16", ref)
