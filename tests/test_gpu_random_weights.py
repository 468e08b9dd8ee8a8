"""Random weights: the device's generator and the host's give the same bits, so a model
drawn on the device (the benchmark's) is the model a folder of the same seed holds."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import TINY_A, TINY_B, seeded_tokens

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.mark.parametrize("n", [1, 255, 4097, 1 << 20])
def test_device_and_host_draw_the_same_bits(n):
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.weights.random_init import normal_deviates, tensor_key

    key = tensor_key(11, f"some.tensor.{n}")
    host = normal_deviates(key, n) * np.float32(0.02)
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    ops.random_normal(out, key, 0.02)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), host.view(np.uint32))
    half = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    ops.random_normal(half, key, 0.02)
    assert torch.equal(half.cpu(), torch.from_numpy(host).to(torch.bfloat16))


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_from_random_is_the_model_a_folder_of_the_same_seed_holds(tmp_path, name, dtype):
    from borrowed_compute_b200 import Engine, StepEntry, write_model_folder
    from borrowed_compute_b200.weights import TensorSource, random_tensors

    cfg = {"A": TINY_A, "B": TINY_B}[name]
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_model_folder(str(tmp_path / "m"), cfg, seed=6, dtype=td)
    src = TensorSource(folder)
    eng_r = Engine.from_random(cfg, 6, dtype=dtype, max_tokens=256)
    drawn = random_tensors(eng_r.model.expected_tensors(), 6, td, "cuda")
    for n in src.names():
        assert torch.equal(drawn[n].cpu(), src.tensor(n)), n
    eng_f = Engine.from_folder(folder, dtype=dtype, max_tokens=256)
    tokens = seeded_tokens(3, 40, cfg["vocab_size"])
    out = []
    for eng in (eng_r, eng_f):
        s = eng.acquire()
        out.append(eng.step([StepEntry(s, tokens, want=tuple(range(40)))]).cpu())
        eng.release(s)
    assert torch.equal(out[0], out[1])
