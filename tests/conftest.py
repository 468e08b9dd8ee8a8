"""Shared fixtures: two tiny configurations that differ in every size and option, seeded
weights, model folders in temporary directories, and the tolerances every comparison uses.

Tolerances are stated once, here.  A float32 engine is held to 1e-4 (1 + max|score|)
against the float64 plain implementation (the reference allows its own GPU 1e-3 (1 +
|score|) against a float64 sum, crates/bc-infer/src/gpu/mod.rs:198).  A bfloat16 engine is
compared with the plain implementation on the same bfloat16-rounded weights and held to
3e-2 (1 + max|score|) on the tiny models (two or three layers).  What they show: about 2e-3
on Tiny A, but up to 2.4e-2 on Tiny B (three layers, a tied head over embeddings of spread 1,
scores up to 40; the largest seen is at a single decoded token late in a replayed batch),
spread evenly over rows and steps as rounding noise is; so neither 1e-2 nor 2e-2 holds there.

Deep models: rounding activations to 8 bits of mantissa five times a layer is independent
noise, so the difference between a bfloat16 and a float32 engine over the same weights grows
with the root of the depth.  Measured on the Llama-3.1-8B shape with random N(0, 0.02)
weights (scores of spread 1.28) against the float32 engine, root mean square of the
difference at 1, 2, 4, 8, 16, 32 layers: 0.013, 0.017, 0.022, 0.030, 0.043, 0.062, which is
2^-8 sqrt(5 layers + 1) times the spread of the scores to within 15 % at every depth (a
relative perturbation of 2^-9 of the embeddings alone gives 0.021 at 32 layers).
``deep_bf16_bounds`` allows one and a half times that for every row's root mean square and
eight times that bound for any single score: a wrong row, page or position moves a row by
the spread of the scores, ten times more.
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

F32_TOL = 1e-4
BF16_TOL = 3e-2


def deep_bf16_bounds(layers: int, ref: np.ndarray):
    """(bound on a row's root-mean-square difference, bound on any one difference) between
    a bfloat16 engine of ``layers`` layers and float32 scores ``ref`` of the same weights."""
    rms = 1.5 * 2.0 ** -8 * float(np.sqrt(5 * layers + 1)) * float(ref.std())
    return rms, 8.0 * rms


def assert_deep_bf16(got: np.ndarray, ref: np.ndarray, layers: int, what: str = "") -> float:
    """Holds bfloat16 scores [rows, vocab] to ``deep_bf16_bounds``; returns the worst row's rms."""
    rms_bound, max_bound = deep_bf16_bounds(layers, ref)
    d = got.astype(np.float64) - ref
    rows = np.sqrt((d * d).mean(axis=1))
    assert rows.max() <= rms_bound, f"{what}: row {int(rows.argmax())} differs by {rows.max():.4g} rms (bound {rms_bound:.4g})"
    assert np.abs(d).max() <= max_bound, f"{what}: a score differs by {np.abs(d).max():.4g} (bound {max_bound:.4g})"
    return float(rows.max())


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # A test marked gpu is skipped where no device is present, whatever -m says.
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny A: grouped-query (4 heads on 2 kv heads), head size implied, widths that are no
# power of two, no frequency scaling, untied head, "half" rotary pairing.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 128, "eos_token_id": 255,
}
# Tiny B: multi-query (1 kv head), explicit head size with heads * head_dim != hidden,
# llama3 frequency scaling that positions pass, tied head, "adjacent" rotary pairing.
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 320, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256, "rope_pairing": "adjacent",
    "eos_token_id": [7, 300],
}
TINY = {"A": TINY_A, "B": TINY_B}


def make_weights(cfg: dict, seed: int, std: float = 0.15, embed_std: float = 1.0, head_std: float = 0.3) -> dict:
    """Seeded float32 weights by tensor name.  The spreads follow the reference's test
    fixture (crates/bc-infer/src/fixtures.rs:7-60: embeddings 1, matrices 0.15, head 0.3,
    norms around 1) so that attention and the gate are far from linear."""
    import plain_llama

    c = plain_llama.read_config(cfg)
    rng = np.random.default_rng(seed)
    qd, kvd = c["heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]

    def mat(rows, cols, s):
        return (rng.standard_normal((rows, cols)) * s).astype(np.float32)

    def vec(n):
        return (1.0 + 0.2 * rng.uniform(-1, 1, n)).astype(np.float32)

    w = {"model.embed_tokens.weight": mat(c["vocab"], c["hidden"], embed_std)}
    for l in range(c["layers"]):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = vec(c["hidden"])
        w[p + "self_attn.q_proj.weight"] = mat(qd, c["hidden"], std)
        w[p + "self_attn.k_proj.weight"] = mat(kvd, c["hidden"], std)
        w[p + "self_attn.v_proj.weight"] = mat(kvd, c["hidden"], std)
        w[p + "self_attn.o_proj.weight"] = mat(c["hidden"], qd, std)
        w[p + "post_attention_layernorm.weight"] = vec(c["hidden"])
        w[p + "mlp.gate_proj.weight"] = mat(c["intermediate"], c["hidden"], std)
        w[p + "mlp.up_proj.weight"] = mat(c["intermediate"], c["hidden"], std)
        w[p + "mlp.down_proj.weight"] = mat(c["hidden"], c["intermediate"], std)
    w["model.norm.weight"] = vec(c["hidden"])
    if not c["tied"]:
        w["lm_head.weight"] = mat(c["vocab"], c["hidden"], head_std)
    return w


def round_bf16(a: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bfloat16 (ties to even), as float32."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(a.shape)


def write_folder(folder: str, cfg: dict, weights: dict, dtype: str) -> str:
    """A model folder holding ``weights`` as float32 or bfloat16."""
    import torch

    from borrowed_compute_b200.weights import write_safetensors

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      {k: torch.from_numpy(np.ascontiguousarray(v)).to(td) for k, v in weights.items()})
    return folder


def weights_as_stored(weights: dict, dtype: str) -> dict:
    """What a folder written with ``dtype`` holds, back as float32 arrays."""
    return weights if dtype == "float32" else {k: round_bf16(v) for k, v in weights.items()}


def tolerance(dtype: str, ref: np.ndarray) -> float:
    return (F32_TOL if dtype == "float32" else BF16_TOL) * (1.0 + float(np.abs(ref).max()))


def seeded_tokens(seed: int, n: int, vocab: int) -> list:
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """(name, dtype) -> (folder, config, weights as the folder stores them)."""
    made = {}

    def get(name: str, dtype: str, seed: int = 5):
        key = (name, dtype, seed)
        if key not in made:
            cfg = TINY[name]
            w = make_weights(cfg, seed)
            folder = write_folder(str(tmp_path_factory.mktemp(f"tiny_{name}_{dtype}")), cfg, w, dtype)
            made[key] = (folder, cfg, weights_as_stored(w, dtype))
        return made[key]

    return get
