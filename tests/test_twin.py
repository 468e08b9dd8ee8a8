"""The plain C++ twin (csrc/twin/plain_twin.cpp) against the plain NumPy implementation:
two restatements of the reference's formulas that share no code must agree, part by part
and on both tiny models; the tiny workloads through the twin are the timed CPU baseline."""

from __future__ import annotations

import time

import numpy as np
import pytest

import plain_llama
from conftest import TINY_A, TINY_B, make_weights, seeded_tokens

twin = pytest.importorskip("borrowed_compute_b200.twin")


def test_parts_agree():
    r = np.random.default_rng(0)
    x, w = r.standard_normal((5, 72)).astype(np.float32), (1 + 0.2 * r.standard_normal(72)).astype(np.float32)
    assert np.abs(twin.rmsnorm(x, w, 1e-6) - plain_llama.rms_norm(x.astype(np.float64), w.astype(np.float64), 1e-6)).max() < 1e-6
    m = r.standard_normal((37, 72)).astype(np.float32)
    assert np.abs(twin.linear(x, m) - x.astype(np.float64) @ m.astype(np.float64).T).max() < 1e-5
    for scaling in (None, TINY_B["rope_scaling"]):
        assert np.array_equal(twin.inv_freq(32, 500000.0, scaling), plain_llama.rope_inv_freq(32, 500000.0, scaling))
    q, k, v = (r.standard_normal(s).astype(np.float32) for s in ((70, 6, 16), (70, 2, 16), (70, 2, 16)))
    freqs = plain_llama.rope_inv_freq(16, 10000.0, None)
    for pairing in ("half", "adjacent"):
        pos = list(range(100, 170))
        assert np.abs(twin.rope(q, pos, freqs, pairing) - plain_llama.rope(q.astype(np.float64), pos, freqs, pairing)).max() < 1e-6
    assert np.abs(twin.attention(q, k, v) - plain_llama.attention(*(a.astype(np.float64) for a in (q, k, v)))).max() < 1e-6
    g, u = r.standard_normal((4, 9)).astype(np.float32), r.standard_normal((4, 9)).astype(np.float32)
    assert np.abs(twin.swiglu(g, u) - g / (1 + np.exp(-g.astype(np.float64))) * u).max() < 1e-6
    # the reference's own sampling case (crates/bc-infer/src/sample.rs:77-89)
    scores = np.array([0.1, 3.0, 2.9, -5.0], dtype=np.float32)
    assert twin.sample(scores, 0.0, 1.0, 0, 0) == 1
    picks = [twin.sample(scores, 1.0, 0.95, 7, i) for i in range(200)]
    assert picks == [plain_llama.sample(scores, 1.0, 0.95, 7, i) for i in range(200)] and 3 not in picks


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B], ids=["A", "B"])
def test_models_agree_and_the_tiny_workloads_are_timed(cfg):
    w = make_weights(cfg, 5)
    model = twin.TwinLlama(cfg, w)
    tokens = seeded_tokens(1, 40, cfg["vocab_size"])
    ref = plain_llama.logits(cfg, w, tokens)
    assert np.abs(model.logits(tokens) - ref).max() <= 1e-4 * (1 + np.abs(ref).max())
    with pytest.raises(ValueError):
        model.logits([cfg["vocab_size"]])
    # the workloads of the two tiny configurations: prompts of 5 / 17 / 1 greedy, of 1 / 9 / 33 / 70 sampled
    lengths, new, sampling = ((5, 17, 1), 8, {}) if cfg is TINY_A else ((1, 9, 33, 70), 16, {"temperature": 0.8, "top_p": 0.9, "seed": 1234567})
    prompts = [seeded_tokens(20 + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)]
    started = time.perf_counter()
    got = [model.generate(p, new, **sampling) for p in prompts]
    seconds = time.perf_counter() - started
    assert got == [plain_llama.generate(cfg, w, p, new, **sampling) for p in prompts]
    assert all(len(o) == new for o in got) and seconds < 60
    stop = got[0][2]
    assert model.generate(prompts[0], new, stops=[stop], **sampling) == got[0][:got[0].index(stop)]
