"""Makes tests/golden/ref_kernels_*.npz: a tiny random Llama scored by the reference's own kernels.

    python tests/golden/make_golden.py --reference <checkout of Harshil089/Borrowed-Compute>

The reference's Rust model code cannot be built without a Rust toolchain, but its GPU
kernel bodies (crates/bc-infer/src/gpu/kernels.h) are plain C.  ref_kernels_driver.cpp
compiles them with g++ under an emulated 32-lane warp and launches them in the order of
crates/bc-infer/src/gpu/mod.rs:454-508.  This script draws the weights, runs the driver
and stores config, seed, tokens and the resulting scores; tests/test_plain.py rebuilds the
same weights from the seed and checks that tests/plain_llama.py scores them alike.

Two cases are made, one per RoPE pairing.  Every inner size is a multiple of 32 because
the reference's product kernel wants that (kernels.h:207; gpu/mod.rs:357).  The per-pair
frequencies come from plain_llama.rope_inv_freq: the reference only divides by stored
factors (model.rs:208-211), so the llama3 rule itself rests on its formula.
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_llama  # noqa: E402

CASES = {
    "adjacent": {
        "config": {
            "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
            "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 96,
            "vocab_size": 80, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": False, "max_position_embeddings": 128, "rope_pairing": "adjacent",
        },
        "seed": 11, "tokens": [3, 79, 14, 0, 41, 41, 7, 65, 22, 9, 50],
    },
    "half": {
        "config": {
            "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
            "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 128,
            "vocab_size": 72, "rope_theta": 500000.0, "rms_norm_eps": 1e-6,
            "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                             "high_freq_factor": 4.0, "original_max_position_embeddings": 8},
            "tie_word_embeddings": True, "max_position_embeddings": 64, "rope_pairing": "half",
        },
        "seed": 12, "tokens": [5, 1, 71, 33, 33, 8, 60, 2, 19, 44, 27, 13, 70],
    },
}


def golden_weights(cfg: dict, seed: int) -> dict:
    """Seeded float32 weights by tensor name; larger than N(0, 0.02) so that attention and
    the gate are far from linear and a wrong formula shows."""
    c = plain_llama.read_config(cfg)
    rng = np.random.default_rng(seed)
    qd, kvd = c["heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]

    def mat(rows, cols, scale):
        return (rng.standard_normal((rows, cols)) * scale).astype(np.float32)

    def vec(n):
        return (1.0 + 0.2 * rng.standard_normal(n)).astype(np.float32)

    w = {"model.embed_tokens.weight": mat(c["vocab"], c["hidden"], 1.0)}
    for l in range(c["layers"]):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = vec(c["hidden"])
        w[p + "self_attn.q_proj.weight"] = mat(qd, c["hidden"], 0.15)
        w[p + "self_attn.k_proj.weight"] = mat(kvd, c["hidden"], 0.15)
        w[p + "self_attn.v_proj.weight"] = mat(kvd, c["hidden"], 0.15)
        w[p + "self_attn.o_proj.weight"] = mat(c["hidden"], qd, 0.15)
        w[p + "post_attention_layernorm.weight"] = vec(c["hidden"])
        w[p + "mlp.gate_proj.weight"] = mat(c["intermediate"], c["hidden"], 0.15)
        w[p + "mlp.up_proj.weight"] = mat(c["intermediate"], c["hidden"], 0.15)
        w[p + "mlp.down_proj.weight"] = mat(c["hidden"], c["intermediate"], 0.15)
    w["model.norm.weight"] = vec(c["hidden"])
    if not c["tied"]:
        w["lm_head.weight"] = mat(c["vocab"], c["hidden"], 0.3)
    return w


def driver_input(cfg: dict, w: dict, tokens) -> bytes:
    c = plain_llama.read_config(cfg)
    neox = 1 if c["pairing"] == "half" else 0
    parts = [
        np.array([c["layers"], c["hidden"], c["heads"], c["kv_heads"], c["head_dim"], c["intermediate"],
                  c["vocab"], len(tokens), neox], dtype="<i4").tobytes(),
        np.array([c["eps"]], dtype="<f4").tobytes(),
        plain_llama.rope_inv_freq(c["head_dim"], c["theta"], c["scaling"]).astype("<f4").tobytes(),
        np.array(tokens, dtype="<i4").tobytes(),
        w["model.embed_tokens.weight"].tobytes(),
    ]
    for l in range(c["layers"]):
        p = f"model.layers.{l}."
        for n in ("input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                  "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"):
            parts.append(w[p + n + ".weight"].tobytes())
    parts.append(w["model.norm.weight"].tobytes())
    parts.append((w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]).tobytes())
    return b"".join(parts)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    inc = os.path.join(args.reference, "crates", "bc-infer", "src", "gpu")
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "driver")
        subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-I", inc,
                        os.path.join(HERE, "ref_kernels_driver.cpp"), "-o", exe], check=True)
        for name, case in CASES.items():
            w = golden_weights(case["config"], case["seed"])
            with open(os.path.join(tmp, "in.bin"), "wb") as f:
                f.write(driver_input(case["config"], w, case["tokens"]))
            subprocess.run([exe, os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")], check=True)
            scores = np.fromfile(os.path.join(tmp, "out.bin"), dtype="<f4").reshape(len(case["tokens"]), -1)
            np.savez_compressed(os.path.join(HERE, f"ref_kernels_{name}.npz"), scores=scores,
                                tokens=np.array(case["tokens"], dtype=np.int32), seed=np.int64(case["seed"]))
            print(name, scores.shape, float(np.abs(scores).max()))


if __name__ == "__main__":
    main()
