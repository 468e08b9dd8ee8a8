"""A sequence of more than 16,384 positions through the engine: more pages than the prompt
kernels keep a list of (256), a decode step cut into more splits than a thread-block cluster
holds (they merge through scratch memory), rotation angles of large positions.  The
reference checks generation past the edge of an attention tile and of the first cache
allocation (crates/bc-infer/src/model.rs:613-674); this is the same question at the far end.

Random weights alone would hide a lost page: among seventeen thousand keys of equal
standing, sixty-four change a result by less than rounding.  So two positions, one in the
fifth page and one past the 256th, hold two tokens whose keys stand out for the query of a
third token, through the pair of dimensions that turns slowest (at these frequencies a
quarter of a radian over the whole sequence), and whose values are large and differ: every
row of the third token gives these two positions nearly all of its weight, and a kernel
that loses either page gives scores that are off by many times the bound (checked on the
host below).  The plain implementation works out the wanted rows alone."""

from __future__ import annotations

import numpy as np
import pytest

import plain_llama
from conftest import make_weights, seeded_tokens, tolerance, weights_as_stored, write_folder

torch = pytest.importorskip("torch")

LENGTH, PROMPT = 17000, 16900
FAR, NEAR = 300, 16450            # the fifth page and the 258th
MARK_FAR, MARK_NEAR, ASKS = 7, 8, 11   # the tokens that are found and the token that looks for them

CONFIGS = {
    # head size 32: pages by cp.async, the mma.sync prompt kernel; a sequence may grow to 24,576 positions, for which
    # a decode step is cut into 64 splits (clusters of eight, their sums through scratch memory)
    "head32": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 128, "num_attention_heads": 4,
               "num_key_value_heads": 2, "intermediate_size": 200, "vocab_size": 301, "rope_theta": 500000.0,
               "rms_norm_eps": 1e-5, "max_position_embeddings": 24576},
    # head size 64: pages by TMA, the tcgen05 prompt kernel; up to 20,480 positions: sixteen splits, one cluster of sixteen
    "head64": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 192, "num_attention_heads": 3,
               "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 264, "vocab_size": 259, "rope_theta": 500000.0,
               "rms_norm_eps": 1e-6, "max_position_embeddings": 20480,
               "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                "original_max_position_embeddings": 8192}},
}


def marked_weights(cfg):
    """Random weights in which token ASKS looks for the tokens MARK_FAR and MARK_NEAR, wherever they stand."""
    c = plain_llama.read_config(cfg)
    w = make_weights(cfg, 9, std=0.05, embed_std=1.0, head_std=0.1)
    hidden, d = c["hidden"], c["head_dim"]
    slow = d - 1 if c["pairing"] == "adjacent" else d // 2 - 1      # a dimension of the slowest pair
    emb = w["model.embed_tokens.weight"]
    for token, column in ((MARK_FAR, 5), (MARK_NEAR, 6), (ASKS, 9)):
        emb[token] = 0.05 * emb[token]
        emb[token, column] = 8.0                                     # after the norm: about sqrt(hidden) in that column
    w["model.layers.0.input_layernorm.weight"][[5, 6, 9]] = 1.0
    w["model.layers.0.self_attn.v_proj.weight"][:, [5, 6]] *= 2.0     # two values that differ and weigh
    gain = (16.0 * np.sqrt(d) / hidden) ** 0.5                       # a score of about 16 where they meet: e^16 against 17,000 others; larger only amplifies the rounding of q and k
    k, q = w["model.layers.0.self_attn.k_proj.weight"], w["model.layers.0.self_attn.q_proj.weight"]
    for g in range(c["kv_heads"]):
        k[g * d + slow, 5] = k[g * d + slow, 6] = gain
    for h in range(c["heads"]):
        q[h * d + slow, 9] = gain
    return w


def sequence(cfg):
    t = seeded_tokens(4, LENGTH, cfg["vocab_size"])
    t = [x if x not in (MARK_FAR, MARK_NEAR, ASKS) else 20 for x in t]
    t[FAR], t[NEAR] = MARK_FAR, MARK_NEAR
    for at in list(range(PROMPT - 40, PROMPT, 3)) + list(range(PROMPT, LENGTH, 2)):
        t[at] = ASKS
    return t


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_sequence_of_seventeen_thousand_positions(name, tmp_path):
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.engine import Engine, StepEntry

    cfg = CONFIGS[name]
    w = marked_weights(cfg)
    t = sequence(cfg)
    wanted = list(range(PROMPT - 40, LENGTH))
    for dtype in ("bfloat16", "float32"):
        stored = weights_as_stored(w, dtype)
        ref = plain_llama.logits(cfg, stored, t, only=wanted)
        folder = write_folder(str(tmp_path / dtype), cfg, w, dtype)
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=cfg["max_position_embeddings"], max_slots=1, max_seq=cfg["max_position_embeddings"])
        if dtype == "bfloat16":
            splits = ops.attention_decode_splits(1, cfg["num_key_value_heads"], eng.cache.slots.max_pages)
            assert splits == (64 if name == "head32" else 16), "the split counts this test is meant to run"
        s = eng.acquire()
        got = []
        cuts = [0, 8192, 16384, PROMPT - 40, PROMPT]                   # the last piece of the prompt is read row by row
        for a, b in zip(cuts, cuts[1:]):
            out = eng.step([StepEntry(s, t[a:b], want=tuple(range(b - a)) if a == PROMPT - 40 else ())])
            if a == PROMPT - 40:
                got.append(out.cpu().numpy())
        for i in range(PROMPT, LENGTH):
            got.append(eng.step([StepEntry(s, [t[i]], want=(0,))]).cpu().numpy())
        eng.release(s)
        eng.cache.slots.check()
        got = np.concatenate(got)
        err = np.abs(got - ref).max(axis=1)
        assert err.max() <= tolerance(dtype, ref), f"{name} {dtype}: first row past the bound is position {wanted[int(np.argmax(err > tolerance(dtype, ref)))]}"


def test_the_marked_positions_hold_the_weight():
    """The construction itself, on the host: a row of the asking token gives the two marked
    positions more than nine tenths of its weight in every head (each at least a tenth), so a lost page shows."""
    for cfg in CONFIGS.values():
        c = plain_llama.read_config(cfg)
        w, t = marked_weights(cfg), sequence(cfg)
        inv = plain_llama.rope_inv_freq(c["head_dim"], c["theta"], c["scaling"])
        x = plain_llama.embed(w["model.embed_tokens.weight"], t)
        n = plain_llama.rms_norm(x, w["model.layers.0.input_layernorm.weight"], c["eps"])
        k = (n @ w["model.layers.0.self_attn.k_proj.weight"].T).reshape(len(t), c["kv_heads"], c["head_dim"])
        k = plain_llama.rope(k, list(range(len(t))), inv, c["pairing"])
        row = LENGTH - 2
        assert t[row] == ASKS
        q = (n[row:row + 1] @ w["model.layers.0.self_attn.q_proj.weight"].T).reshape(1, c["heads"], c["head_dim"])
        q = plain_llama.rope(q, [row], inv, c["pairing"])
        for h in range(c["heads"]):
            s = k[: row + 1, h // (c["heads"] // c["kv_heads"])] @ q[0, h] / np.sqrt(c["head_dim"])
            p = np.exp(s - s.max())
            p /= p.sum()
            assert p[FAR] + p[NEAR] > 0.9 and min(p[FAR], p[NEAR]) > 0.1, (h, p[FAR], p[NEAR])
        # What losing either position would do to the scores of that row: many times the bound.
        ref = plain_llama.logits(cfg, w, t, only=[row])
        for at in (FAR, NEAR):
            without = list(t)
            without[at] = 20
            assert np.abs(plain_llama.logits(cfg, w, without, only=[row]) - ref).max() > 10 * tolerance("bfloat16", ref)


@pytest.mark.gpu
def test_captured_steps_change_when_a_sequence_crosses_a_bound(tmp_path):
    """A captured decode step is made for a bound on the positions it reaches (a power of
    two from 4,096 on), by which the attention plans its splits.  Two sequences, one of which
    crosses 4,096 while the other stays short: the steps before, at and after the crossing,
    staged ahead and fed from the device as the generation loop does, give the scores of
    steps that are not captured, to the bit (at these lengths both ways cut the same)."""
    from borrowed_compute_b200.engine import Engine, StepEntry

    cfg = CONFIGS["head64"]
    w = make_weights(cfg, 3, std=0.05, embed_std=1.0, head_std=0.1)
    folder = write_folder(str(tmp_path / "m"), cfg, w, "bfloat16")
    long, short = seeded_tokens(5, 4110, cfg["vocab_size"]), seeded_tokens(6, 60, cfg["vocab_size"])
    runs = {}
    for captured in (True, False):
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=4352, max_slots=2, max_seq=cfg["max_position_embeddings"])
        eng.use_graphs = eng.use_graphs and captured
        a, b = eng.acquire(), eng.acquire()
        eng.step([StepEntry(a, long[:4090], want=()), StepEntry(b, short[:40], want=())])
        got = []
        for i in range(20):
            feed = (long[4090 + i], short[40 + i])
            if captured and i > 0 and eng.can_step_again((a, b)):
                eng.last_graph.views["tokens"][:2].copy_(torch.tensor(feed, dtype=torch.int32))   # as a sampler on the device would
                got.append(eng.step_again().cpu().numpy())
            else:
                assert not captured or i == 0 or 4090 + i == 4096, f"step {i} was not staged"   # the step that crosses starts anew
                got.append(eng.step([StepEntry(a, (feed[0],), want=(0,)), StepEntry(b, (feed[1],), want=(0,))]).cpu().numpy())
        if captured:
            assert sorted(eng._graphs) == [(2, 4096), (2, min(8192, eng.max_seq))]
        eng.release(a), eng.release(b)
        eng.cache.slots.check()
        runs[captured] = np.stack(got)
    assert np.array_equal(runs[True], runs[False])
    ref = plain_llama.logits(cfg, weights_as_stored(w, "bfloat16"), long, only=list(range(4090, 4110)))
    assert np.abs(runs[True][:, 0] - ref).max() <= tolerance("bfloat16", ref)
