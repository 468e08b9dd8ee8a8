"""A plain, slow Llama dense decoder in NumPy: whole sequences, no cache, one function a part.

This is the oracle of the test suite.  It shares no code with the package under test: it
reads a config dict and a dict of arrays keyed by tensor name, and recomputes every
position of a sequence from scratch.  Every function restates one formula of the
reference engine (Harshil089/Borrowed-Compute) and cites where that formula lives, by the
file's path inside that project.

The arithmetic runs in float64 unless ``dtype`` says otherwise, so that a float32 engine is
compared against something more exact than itself.
"""

from __future__ import annotations

import math

import numpy as np

MASK64 = (1 << 64) - 1


# --------------------------------------------------------------------------- configuration

def read_config(cfg: dict) -> dict:
    """The sizes and constants of one model, with the defaults the reference applies.

    crates/bc-infer/src/model.rs:44-70: kv heads default to the head count (60), the head
    size to ``n_embd / n_head`` (51), the rope base to 10000 (63), eps to 1e-5 (65) and the
    context to 4096 (67).  The keys are config.json's names for the same quantities.
    """
    heads = int(cfg["num_attention_heads"])
    hidden = int(cfg["hidden_size"])
    out = {
        "layers": int(cfg["num_hidden_layers"]),
        "hidden": hidden,
        "heads": heads,
        "kv_heads": int(cfg.get("num_key_value_heads") or heads),
        "head_dim": int(cfg.get("head_dim") or hidden // heads),
        "intermediate": int(cfg["intermediate_size"]),
        "vocab": int(cfg["vocab_size"]),
        "theta": float(cfg.get("rope_theta", 10000.0)),
        "scaling": cfg.get("rope_scaling"),
        "eps": float(cfg.get("rms_norm_eps", 1e-5)),
        "tied": bool(cfg.get("tie_word_embeddings", False)),
        "context": int(cfg.get("max_position_embeddings", 4096)),
        # model.rs:36-37,64: which two dimensions of a head form a rotated pair.
        "pairing": cfg.get("rope_pairing", "half"),
    }
    return out


# --------------------------------------------------------------------------------- the parts

def embed(table: np.ndarray, tokens) -> np.ndarray:
    """Row ``t`` of the embedding table for every token (model.rs:270-280)."""
    rows = []
    for t in tokens:
        if not 0 <= int(t) < table.shape[0]:
            raise ValueError(f"token {t} is outside the vocabulary")
        rows.append(table[int(t)])
    return np.stack(rows).astype(np.float64)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """``x * (1/sqrt(mean(x^2) + eps)) * w`` row by row (model.rs:381-389;
    gpu/kernels.h:226-233): eps inside the root, the weight applied after the scale."""
    ms = (x * x).sum(axis=-1, keepdims=True) / x.shape[-1]
    return x * (1.0 / np.sqrt(ms + eps)) * w


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> np.ndarray:
    """One frequency per rotated pair: ``theta^(-2i/d) / factor_i`` (model.rs:208-211).

    The reference reads ``factor_i`` from a stored tensor; here it is derived from the
    llama3 scaling rule: wavelengths shorter than ``orig/high`` keep their frequency,
    longer than ``orig/low`` are divided by ``factor``, and those between blend the two
    linearly in ``orig/wavelength``.  The result is rounded to float32 once, because the
    engine stores it so and the angle is a float32 product (kernels.h:241).
    """
    half = head_dim // 2
    out = np.empty(half, dtype=np.float64)
    for i in range(half):
        f = theta ** (-2.0 * i / head_dim)
        if scaling is not None:
            s = float(scaling["factor"])
            lo = float(scaling["low_freq_factor"])
            hi = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / hi:
                pass
            elif wavelen > orig / lo:
                f = f / s
            else:
                t = (orig / wavelen - lo) / (hi - lo)
                f = (1.0 - t) * f / s + t * f
        out[i] = f
    return out.astype(np.float32)


def rope(x: np.ndarray, positions, inv_freq: np.ndarray, pairing: str) -> np.ndarray:
    """Rotates every head of ``x[row, head, dim]`` by ``position * inv_freq[i]``
    (model.rs:391-403; kernels.h:237-248).  The angle is the float32 product of the
    position and the float32 frequency, as in the reference; pairs are ``(2i, 2i+1)``
    ("adjacent") or ``(i, i + d/2)`` ("half")."""
    rows, heads, d = x.shape
    half = d // 2
    out = x.copy()
    for r in range(rows):
        ang = (np.float32(positions[r]) * inv_freq.astype(np.float32)).astype(np.float64)
        cos, sin = np.cos(ang), np.sin(ang)
        for i in range(half):
            a, b = (i, i + half) if pairing == "half" else (2 * i, 2 * i + 1)
            x0, x1 = x[r, :, a], x[r, :, b]
            out[r, :, a] = x0 * cos[i] - x1 * sin[i]
            out[r, :, b] = x0 * sin[i] + x1 * cos[i]
    return out


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, only=None) -> np.ndarray:
    """Causal grouped-query attention over one whole sequence (model.rs:448-481).

    ``q[row, head, d]``, ``k, v[row, kv_head, d]``.  Row ``i`` sees rows ``0..i``; head
    ``h`` reads kv head ``h // (heads / kv_heads)`` (463); scores are scaled by
    ``1/sqrt(d)`` (451), the maximum is subtracted before the exponential (466-470).
    ``only``: the rows whose result is wanted; then ``q`` holds these rows alone, in this
    order, and so does the result (a long sequence of which the test reads the end).
    """
    heads, d = q.shape[1], q.shape[2]
    group = heads // k.shape[1]
    scale = 1.0 / math.sqrt(d)
    out = np.zeros_like(q)
    for at, i in enumerate(range(q.shape[0]) if only is None else only):
        for h in range(heads):
            g = h // group
            s = (k[: i + 1, g, :] @ q[at, h, :]) * scale
            p = np.exp(s - s.max())
            out[at, h, :] = (p / p.sum()) @ v[: i + 1, g, :]
    return out


def swiglu(x: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    """``down( g/(1+e^-g) * u )`` with ``g = x gate^T`` and ``u = x up^T``
    (model.rs:341-344; kernels.h:330)."""
    g = x @ gate.T
    u = x @ up.T
    return (g / (1.0 + np.exp(-g)) * u) @ down.T


def layer(x, w, prefix, c, positions, inv_freq, only=None):
    """One pre-norm block (model.rs:323-345): attention and feed-forward, each added to
    the stream it read through a norm.  ``only``: rows whose result is wanted (every row
    still gives its key and value); the result then holds these rows alone."""
    rows = x.shape[0]
    n = rms_norm(x, w[prefix + "input_layernorm.weight"], c["eps"])
    k = (n @ w[prefix + "self_attn.k_proj.weight"].T).reshape(rows, c["kv_heads"], c["head_dim"])
    v = (n @ w[prefix + "self_attn.v_proj.weight"].T).reshape(rows, c["kv_heads"], c["head_dim"])
    k = rope(k, positions, inv_freq, c["pairing"])
    if only is not None:
        x, n, rows = x[list(only)], n[list(only)], len(only)
        positions = [positions[i] for i in only]
    q = (n @ w[prefix + "self_attn.q_proj.weight"].T).reshape(rows, c["heads"], c["head_dim"])
    q = rope(q, positions, inv_freq, c["pairing"])
    att = attention(q, k, v, only).reshape(rows, c["heads"] * c["head_dim"])
    x = x + att @ w[prefix + "self_attn.o_proj.weight"].T
    n = rms_norm(x, w[prefix + "post_attention_layernorm.weight"], c["eps"])
    return x + swiglu(
        n,
        w[prefix + "mlp.gate_proj.weight"],
        w[prefix + "mlp.up_proj.weight"],
        w[prefix + "mlp.down_proj.weight"],
    )


def head(x, w, c):
    """Final norm and output product; a tied model scores against the embedding table
    (model.rs:200,361-370)."""
    n = rms_norm(x, w["model.norm.weight"], c["eps"])
    out = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]
    return n @ out.T


def logits(cfg: dict, weights: dict, tokens, dtype=np.float64, only=None) -> np.ndarray:
    """Scores after every token of one sequence fed from position 0: ``[len, vocab]``
    (the sequence of crates/bc-infer/src/lib.rs:50-54: embed, layers, head).  ``only``:
    the positions whose scores are wanted; the last layer and the head then run for these
    alone (every layer before it runs whole, since later rows read its keys and values)."""
    c = read_config(cfg)
    w = {k: np.asarray(v).astype(dtype) for k, v in weights.items()}
    positions = list(range(len(tokens)))
    inv_freq = rope_inv_freq(c["head_dim"], c["theta"], c["scaling"])
    x = embed(w["model.embed_tokens.weight"], tokens).astype(dtype)
    for l in range(c["layers"]):
        x = layer(x, w, f"model.layers.{l}.", c, positions, inv_freq, only if l == c["layers"] - 1 else None)
    return head(x, w, c)


# ---------------------------------------------------------------------------------- sampling

def argmax(scores) -> int:
    """The first largest score wins (crates/bc-infer/src/sample.rs:24-32)."""
    best = 0
    for i, s in enumerate(scores):
        if s > scores[best]:
            best = i
    return best


def uniform(seed: int) -> float:
    """splitmix64's finaliser; the top 24 bits over 2^24 (sample.rs:64-71)."""
    z = (seed + 0x9E3779B97F4A7C15) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return float(z >> 40) / float(1 << 24)


def nucleus(scores, temperature: float, top_p: float):
    """The kept tokens, in drawing order, with their weights (sample.rs:39-52):
    ``w = e^((s - max)/T)``, sorted descending (stable, so ties keep ascending ids), cut
    to the shortest prefix whose share of the total reaches ``top_p``."""
    s = np.asarray(scores, dtype=np.float64)
    w = np.exp((s - s.max()) / temperature)
    total = w.sum()
    order = sorted(range(len(w)), key=lambda i: -w[i])
    keep, mass = 0, 0.0
    for i in order:
        keep += 1
        mass += w[i] / total
        if mass >= top_p:
            break
    order = order[: max(keep, 1)]
    return order, w[order]


def sample(scores, temperature: float, top_p: float, seed: int, step: int) -> int:
    """One draw (sample.rs:35-62): greedy at ``temperature <= 0``; else a uniform number
    from ``seed ^ step * 0x9e3779b97f4a7c15`` scaled to the kept mass, walked down the
    kept list."""
    if temperature <= 0.0:
        return argmax(scores)
    order, w = nucleus(scores, temperature, top_p)
    r = uniform((seed ^ ((step * 0x9E3779B97F4A7C15) & MASK64)) & MASK64) * w.sum()
    for i, wi in zip(order, w):
        r -= wi
        if r <= 0.0:
            return int(i)
    return int(order[0])


def generate(cfg, weights, prompt, max_tokens, temperature=0.0, top_p=1.0, seed=0, stops=()):
    """Greedy or sampled continuation of one prompt by recomputing the whole sequence
    each step (the loop of crates/bc-infer/examples/generate.rs:33-44; a stop id ends the
    text and is not part of it, crates/bc-mesh/src/llm.rs:549-552; the draw's step is the
    position of the row sampled, crates/bc-mesh/src/engine.rs:347-350)."""
    seq = list(prompt)
    out = []
    while len(out) < max_tokens:
        row = logits(cfg, weights, seq)[-1]
        tok = sample(row, temperature, top_p, seed, len(seq) - 1)
        if tok in stops:
            break
        out.append(tok)
        seq.append(tok)
    return out
