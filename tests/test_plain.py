"""The plain implementation itself: against the reference's own kernels (golden files made
by tests/golden/make_golden.py), against the reference's sampling test, and for the
properties the reference tests of its rotary encoding."""

from __future__ import annotations

import math
import os
import sys

import numpy as np

import plain_llama

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402


def test_plain_matches_the_reference_kernels():
    """The golden scores were computed by the reference's kernel bodies
    (crates/bc-infer/src/gpu/kernels.h) in float32; the plain implementation works in
    float64, so they agree to float32 rounding of scores of size ~10."""
    for name, case in make_golden.CASES.items():
        g = np.load(os.path.join(HERE, "golden", f"ref_kernels_{name}.npz"))
        assert list(g["tokens"]) == case["tokens"] and int(g["seed"]) == case["seed"]
        w = make_golden.golden_weights(case["config"], case["seed"])
        got = plain_llama.logits(case["config"], w, case["tokens"])
        ref = g["scores"].astype(np.float64)
        assert got.shape == ref.shape
        assert np.abs(got - ref).max() <= 2e-6 * (1 + np.abs(ref).max()), name


def test_sampling_on_the_reference_case():
    """crates/bc-infer/src/sample.rs:77-89."""
    scores = [0.1, 3.0, 2.9, -5.0]
    assert plain_llama.sample(scores, 0.0, 1.0, 0, 0) == 1
    assert all(plain_llama.sample(scores, 1.0, 0.01, 7, i) == 1 for i in range(20))
    picks = [plain_llama.sample(scores, 1.0, 0.95, 7, i) for i in range(200)]
    assert 1 in picks and 2 in picks and 3 not in picks
    assert picks == [plain_llama.sample(scores, 1.0, 0.95, 7, i) for i in range(200)]


def test_uniform_is_splitmix64():
    # splitmix64 of seed 0: the first output of the well-known generator is 0xe220a8397b1dcdaf.
    z = 0xE220A8397B1DCDAF
    assert plain_llama.uniform(0) == float(z >> 40) / float(1 << 24)
    assert 0.0 <= plain_llama.uniform(12345) < 1.0


def test_argmax_first_largest():
    assert plain_llama.argmax([1.0, 5.0, 5.0, 2.0]) == 1
    assert plain_llama.argmax([-3.0]) == 0


def test_rope_rotates_pairs_by_position():
    """crates/bc-infer/src/model.rs:676-688: position 0 is the identity, position 1 turns
    the first pair by one radian, rotations keep length."""
    inv = plain_llama.rope_inv_freq(4, 10000.0, None)
    assert inv[0] == 1.0
    x = np.array([[[1.0, 0.0, 1.0, 0.0]]])
    assert np.array_equal(plain_llama.rope(x, [0], inv, "adjacent"), x)
    y = plain_llama.rope(x, [1], inv, "adjacent")
    assert abs(y[0, 0, 0] - math.cos(1.0)) < 1e-12 and abs(y[0, 0, 1] - math.sin(1.0)) < 1e-12
    z = plain_llama.rope(np.array([[[1.0, 1.0, 0.0, 0.0]]]), [1], inv, "half")
    assert abs(z[0, 0, 0] - math.cos(1.0)) < 1e-12 and abs(z[0, 0, 2] - math.sin(1.0)) < 1e-12
    r = np.random.default_rng(0).standard_normal((3, 2, 8))
    for pairing in ("half", "adjacent"):
        out = plain_llama.rope(r, [5, 100, 7], plain_llama.rope_inv_freq(8, 500000.0, None), pairing)
        assert np.allclose((out ** 2).sum(-1), (r ** 2).sum(-1))


def test_llama3_scaling_leaves_high_frequencies_and_slows_low_ones():
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    plain = plain_llama.rope_inv_freq(128, 500000.0, None).astype(np.float64)
    scaled = plain_llama.rope_inv_freq(128, 500000.0, scaling).astype(np.float64)
    wavelen = 2 * math.pi / plain
    assert np.array_equal(scaled[wavelen < 8192 / 4], plain[wavelen < 8192 / 4])
    low = wavelen > 8192
    assert low.any() and np.allclose(scaled[low], plain[low] / 8.0, rtol=1e-6)
    mid = ~low & ~(wavelen < 8192 / 4)
    assert mid.any() and np.all(scaled[mid] < plain[mid]) and np.all(scaled[mid] > plain[mid] / 8.0)


def test_attention_is_causal_and_grouped():
    r = np.random.default_rng(1)
    q, k, v = r.standard_normal((5, 4, 8)), r.standard_normal((5, 2, 8)), r.standard_normal((5, 2, 8))
    out = plain_llama.attention(q, k, v)
    assert np.allclose(out[0], np.repeat(v[0], 2, axis=0))          # the first row sees only itself
    k2, v2 = k.copy(), v.copy()
    k2[4], v2[4] = 100.0, -100.0                                     # the future changes no earlier row
    assert np.array_equal(plain_llama.attention(q, k2, v2)[:4], out[:4])
    v3 = v.copy()
    v3[:, 1] += 1.0                                                  # kv head 1 serves heads 2 and 3 only
    d = plain_llama.attention(q, k, v3) - out
    assert np.allclose(d[:, :2], 0.0) and np.allclose(d[:, 2:], 1.0)


def test_generate_stops_without_emitting():
    cfg = make_golden.CASES["adjacent"]["config"]
    w = make_golden.golden_weights(cfg, 3)
    free = plain_llama.generate(cfg, w, [1, 2, 3], 6)
    assert len(free) == 6
    stopped = plain_llama.generate(cfg, w, [1, 2, 3], 6, stops=(free[2],))
    assert stopped == free[:free.index(free[2])]


def test_wanted_rows_alone_give_the_rows_of_the_whole():
    from conftest import TINY_B, make_weights

    w = make_weights(TINY_B, 4)
    tokens = [int(t) for t in np.random.default_rng(0).integers(0, TINY_B["vocab_size"], 23)]
    whole = plain_llama.logits(TINY_B, w, tokens)
    some = plain_llama.logits(TINY_B, w, tokens, only=[22, 3, 17])
    assert some.shape == (3, TINY_B["vocab_size"])
    assert np.allclose(some, whole[[22, 3, 17]], rtol=0, atol=1e-11)   # the library's products round by their shapes
