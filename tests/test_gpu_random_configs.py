"""Configurations drawn at random (every size and option: head sizes 16 to 128, heads and
groups, widths and vocabularies of any size, layers, eps, theta, pairing, tied head, llama3
scaling) under random ragged traffic: prompts in one step, a continuation chunk for some
requests, single tokens while the shorter requests end, slots given back and taken again.
The float32 engine is held to the plain implementation, the bfloat16 engine to the plain
implementation with bf16-stored weights."""

from __future__ import annotations

import numpy as np
import pytest

import plain_llama
from conftest import make_weights, tolerance, weights_as_stored, write_folder

pytestmark = pytest.mark.gpu


def draw_config(r):
    D = int(r.choice([16, 32, 48, 64, 128]))
    G = int(r.choice([1, 2, 3, 4]))
    H = G * int(r.choice([1, 2, 3, 4, 5, 8]))
    cfg = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": int(r.integers(1, 4)), "hidden_size": 8 * int(r.integers(4, 60)),
           "num_attention_heads": H, "num_key_value_heads": G, "head_dim": D, "intermediate_size": 8 * int(r.integers(4, 120)),
           "vocab_size": int(r.integers(50, 2000)), "rope_theta": float(r.choice([10000.0, 500000.0])),
           "rms_norm_eps": float(r.choice([1e-5, 1e-6])), "max_position_embeddings": 1024, "tie_word_embeddings": bool(r.integers(0, 2)),
           "rope_pairing": str(r.choice(["half", "adjacent"]))}
    if r.integers(0, 3) == 0:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 128}
    return cfg


@pytest.mark.parametrize("seed", [3, 14, 15, 92, 65, 35])
def test_random_configuration_under_random_traffic(seed, tmp_path):
    from borrowed_compute_b200.engine import Engine, StepEntry

    r = np.random.default_rng(seed)
    cfg = draw_config(r)
    V = cfg["vocab_size"]
    w = make_weights(cfg, seed, std=0.04, embed_std=1.0, head_std=0.1)
    n = int(r.integers(2, 5))
    lens = [int(r.choice([1, 2, 7, 33, 64, 65, 130, 200, 300])) for _ in range(n)]
    extra = [int(r.choice([0, 0, 3, 70, 150])) for _ in range(n)]
    single = [int(r.integers(0, 12)) for _ in range(n)]
    toks = [[int(x) for x in r.integers(0, V, lens[i] + extra[i] + single[i])] for i in range(n)]
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(write_folder(str(tmp_path / dtype), cfg, w, dtype), dtype=dtype, max_tokens=4096, max_slots=n)
        stored = weights_as_stored(w, dtype)
        refs = [plain_llama.logits(cfg, stored, t, dtype=np.float32) for t in toks]
        for round_ in range(2):                           # the second round takes the slots the first gave back
            slots = [eng.acquire() for _ in range(n)]
            got = [[] for _ in range(n)]
            out = eng.step([StepEntry(slots[i], toks[i][:lens[i]], want=tuple(range(lens[i]))) for i in range(n)]).cpu().numpy()
            at, row = list(lens), 0
            for i in range(n):
                got[i].append(out[row:row + lens[i]])
                row += lens[i]
            cont = [i for i in range(n) if extra[i] > 0]
            if cont:
                out = eng.step([StepEntry(slots[i], toks[i][at[i]:at[i] + extra[i]], want=tuple(range(extra[i]))) for i in cont]).cpu().numpy()
                row = 0
                for i in cont:
                    got[i].append(out[row:row + extra[i]])
                    row += extra[i]
                    at[i] += extra[i]
            live = [i for i in range(n) if at[i] < len(toks[i])]
            for i in range(n):
                if i not in live:
                    eng.release(slots[i])                 # nothing left to decode
            while live:
                out = eng.step([StepEntry(slots[i], [toks[i][at[i]]], want=(0,)) for i in live]).cpu().numpy()
                for k, i in enumerate(live):
                    got[i].append(out[k:k + 1])
                    at[i] += 1
                    if at[i] == len(toks[i]):
                        eng.release(slots[i])             # the shorter requests end earlier
                live = [i for i in live if at[i] < len(toks[i])]
            for i in range(n):
                mine = np.concatenate(got[i])
                tol = 2 * tolerance(dtype, refs[i])       # the plain run is float32 here: allow for its own rounding too
                err = float(np.abs(mine - refs[i]).max())
                assert err <= tol, f"seed {seed} {cfg} {dtype} round {round_} request {i}: error {err:.3e} over {tol:.3e}"
            eng.cache.slots.check()
            assert eng.cache.slots.live() == []
