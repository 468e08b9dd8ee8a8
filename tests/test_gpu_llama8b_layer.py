"""One layer of the Llama-3.1-8B shape (hidden 4096, 32 heads on 8 kv heads of 128, feed-forward
14336, llama3 scaling with factor 8) with a vocabulary that is no power of two: the sizes the
benchmark runs, held to the plain implementation and to each other under the three cuts."""

from __future__ import annotations

import numpy as np
import pytest

import plain_llama
from conftest import make_weights, seeded_tokens, tolerance, weights_as_stored, write_folder

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 8072, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}


@pytest.fixture(scope="module")
def layer(tmp_path_factory):
    w = make_weights(CONFIG, 21, std=0.02, embed_std=1.0, head_std=0.05)
    # Sharpen attention: with N(0, 0.02) projections every score is near zero and a wrong
    # position would hardly show.
    w["model.layers.0.self_attn.q_proj.weight"] *= 4.0
    w["model.layers.0.self_attn.k_proj.weight"] *= 4.0
    folders = {d: write_folder(str(tmp_path_factory.mktemp(f"l8b_{d}")), CONFIG, w, d) for d in ("float32", "bfloat16")}
    return folders, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_of_the_8b_shape(layer, dtype):
    from borrowed_compute_b200.engine import Engine, StepEntry

    folders, w = layer
    eng = Engine.from_folder(folders[dtype], dtype=dtype, max_tokens=1024, max_slots=4)
    a, b = seeded_tokens(1, 150, CONFIG["vocab_size"]), seeded_tokens(2, 70, CONFIG["vocab_size"])
    stored = weights_as_stored(w, dtype)
    ref_a = plain_llama.logits(CONFIG, stored, a, dtype=np.float32)[-40:]
    ref_b = plain_llama.logits(CONFIG, stored, b, dtype=np.float32)[-40:]
    # The plain run is float32 here (its matrices are large); allow for its own rounding too.
    tol = 2 * tolerance(dtype, ref_a)

    def want(n, k=40):
        return tuple(range(n - k, n))

    s = eng.acquire()
    whole = eng.step([StepEntry(s, a, want=want(len(a)))]).cpu().numpy()
    eng.release(s)
    assert np.abs(whole - ref_a).max() <= tol, "whole prompt"
    # the last 32 tokens one by one (through the captured decode graph)
    s = eng.acquire()
    cut = len(a) - 32
    head = eng.step([StepEntry(s, a[:cut], want=want(cut, 8))]).cpu().numpy()
    tail = np.concatenate([eng.step([StepEntry(s, [t], want=(0,))]).cpu().numpy() for t in a[cut:]])
    eng.release(s)
    decoded = np.concatenate([head, tail])
    assert np.abs(decoded - ref_a).max() <= tol, "prompt then 32 single tokens"
    # both requests in one batch, the shorter ending earlier
    sa, sb = eng.acquire(), eng.acquire()
    first = eng.step([StepEntry(sa, a[:-5], want=want(len(a) - 5, 35)), StepEntry(sb, b[:-3], want=want(len(b) - 3, 37))]).cpu().numpy()
    got_a, got_b = [first[:35]], [first[35:]]
    for i in range(5):
        entries = [StepEntry(sa, [a[len(a) - 5 + i]], want=(0,))] + ([StepEntry(sb, [b[len(b) - 3 + i]], want=(0,))] if i < 3 else [])
        out = eng.step(entries).cpu().numpy()
        got_a.append(out[:1])
        if i < 3:
            got_b.append(out[1:])
        if i == 2:
            eng.release(sb)
    eng.release(sa)
    assert np.abs(np.concatenate(got_a) - ref_a).max() <= tol and np.abs(np.concatenate(got_b) - ref_b).max() <= tol, "batch"
    if dtype == "float32":
        assert np.array_equal(decoded, whole) and np.array_equal(np.concatenate(got_a), whole), "float32 cuts must agree to the bit"
    from borrowed_compute_b200 import ops
    assert ops.gemm_tc_status() == 0
