"""Decode and prefill throughput of the Llama-3.1-8B shape on one B200, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]
                    [--no-points] [--no-breakdown]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  ``value`` is decoded
tokens a second timed on the device (CUDA events around K steps, after W warm-up steps);
``e2e`` is the same through the Python entry point (``Local.generate``: host token ids in,
host token ids out every step); ``prefill`` is one 2,048-token prompt; ``roofline`` sets the
decode step's mandatory bytes (every weight once, the live requests' cache once) against the
measured copy bandwidth.  ``points`` adds decoding at batch 1 and 64 (device-timed and end to
end) and two more workloads of other shapes: the Llama-2-13B shape (one kv head a head) with
16 prompts of unequal lengths, and the Llama-3.2-3B shape (tied head) at batch 64 sampled at
temperature 1.0 through the entry point, and the two tiny workloads on the device and on the
library's plain C++ twin on the host (the CPU baseline).  ``classes`` times every kernel class of one decode
step and one prompt step launch by launch and sets each against its own bytes or operations.
``checked`` says that the tokens of the end-to-end run equal those of the same prompts
stepped without captured graphs; the line is not printed otherwise.  Every decode step
streams all weights (16 GB), far more than the 126 MB L2, so nothing is flushed between
iterations.

The reference (Harshil089/Borrowed-Compute) is a Rust workspace; no Rust toolchain exists
here, so ``--impl reference`` reports itself unavailable.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _llama3_scaling(factor: float) -> dict:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}


# The headline: the Llama-3.1-8B shape.
CONFIG_8B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": _llama3_scaling(8.0), "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}
# The Llama-2-13B shape: every head has a kv head of its own.
CONFIG_13B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40,
    "num_key_value_heads": 40, "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
# The Llama-3.2-3B shape: the head is the embedding table.
CONFIG_3B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 28, "hidden_size": 3072, "num_attention_heads": 24,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": _llama3_scaling(32.0), "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 16384,
}
# The two tiny configurations, which differ in every size and option; their workloads are timed
# against the library's plain C++ twin on the host.
CONFIG_TINY_A = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 128,
}
CONFIG_TINY_B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 4, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 320, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256,
}
CONTEXT = 8192
PROMPT = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


E2E_SETTLE_PASSES = 24   # decode passes after a prompt before the end-to-end clock starts (see end_to_end)


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        if "bf16_tflops_sustained" in d:
            out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        return out
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc, self.thread = [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not mhz:
            return None
        return {"sm_mhz": int(statistics.median(mhz)), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


# ------------------------------------------------------------------------ bytes and operations
def model_numbers(cfg: dict, layers: int) -> dict:
    E, H, G, D, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                        cfg["intermediate_size"], cfg["vocab_size"])
    qkv, o, gate_up, down = E * (H + 2 * G) * D, H * D * E, 2 * E * F, E * F
    return {"qkv": qkv, "o": o, "gate_up": gate_up, "down": down, "layer_params": qkv + o + gate_up + down, "head_params": V * E,
            "norm_params": (2 * layers + 1) * E, "kv_bytes_per_token": layers * 2 * G * D * 2, "E": E, "H": H, "G": G, "D": D, "F": F, "V": V}


def decode_bytes(cfg, layers, batch, cached_tokens) -> float:
    """What a decode step has to read: every weight it uses once (a tied head is the
    embedding table, read once as the head), the norms, the batch's embedding rows, and
    the cache of the live requests (``cached_tokens`` positions in all)."""
    n = model_numbers(cfg, layers)
    weights = 2.0 * (layers * n["layer_params"] + n["head_params"]) + 4.0 * n["norm_params"] + 2.0 * batch * n["E"]
    return weights + float(cached_tokens) * n["kv_bytes_per_token"]


def prefill_flops(cfg, layers, lengths) -> float:
    """Operations of one prompt step over sequences of ``lengths`` tokens, scores at each one's last token."""
    n = model_numbers(cfg, layers)
    tokens = sum(lengths)
    linear = 2.0 * tokens * layers * n["layer_params"]
    attention = sum(layers * 2.0 * 2.0 * n["H"] * n["D"] * t * (t + 1) / 2.0 for t in lengths)
    return linear + attention + 2.0 * n["head_params"] * len(lengths)


def class_costs(cfg, layers, batch, cached_tokens, prompt_tokens) -> dict:
    """What each kernel class of a decode step has to move (bytes) and of a one-sequence
    prompt step has to compute (operations; bytes for the classes that only move data)."""
    n = model_numbers(cfg, layers)
    E, H, G, D, F, V = n["E"], n["H"], n["G"], n["D"], n["F"], n["V"]
    B, T = batch, prompt_tokens
    qkv_w = (H + 2 * G) * D
    decode = {
        "embedding": B * E * 6.0,
        "norm": (2 * layers + 1) * (B * E * 6.0 + E * 4.0),
        "qkv product": layers * (2.0 * n["qkv"] + 2.0 * B * (E + qkv_w)),
        "attention": float(cached_tokens) * n["kv_bytes_per_token"] + layers * 2.0 * B * (qkv_w + H * D),
        "output product": layers * (2.0 * n["o"] + B * (2.0 * H * D + 8.0 * E)),
        "gate/up product": layers * (2.0 * n["gate_up"] + 2.0 * B * (E + F)),
        "down product": layers * (2.0 * n["down"] + B * (2.0 * F + 8.0 * E)),
        "head product": 2.0 * n["head_params"] + B * (2.0 * E + 4.0 * V),
        "sampling": B * V * 4.0,
    }
    prefill = {
        "embedding": ("bytes", T * E * 6.0),
        "norm": ("bytes", 2 * layers * T * E * 6.0 + E * 6.0),
        "qkv product": ("flops", layers * 2.0 * T * n["qkv"]),
        "rotary + append": ("bytes", layers * 2.0 * T * (2.0 * (H + G) * D + 2.0 * G * D + 2.0 * G * D)),
        "attention": ("flops", layers * 4.0 * H * D * T * (T + 1) / 2.0),
        "output product": ("flops", layers * 2.0 * T * n["o"]),
        "gate/up product": ("flops", layers * 2.0 * T * n["gate_up"]),
        "down product": ("flops", layers * 2.0 * T * n["down"]),
        "head product": ("bytes", 2.0 * n["head_params"]),
    }
    return {"decode": decode, "prefill": prefill}


# ------------------------------------------------------------------------------- measuring
def free_device_memory():
    import torch

    gc.collect()
    torch.cuda.empty_cache()


def timed_decode(eng, prompts, steps, warmup, rng, vocab, sample_clocks=False, prompts_a_step=8):
    """Device time of ``steps`` decode steps of the given sequences after their prompts.
    Returns also the prompt step's time when all prompts go in one step."""
    import torch

    from borrowed_compute_b200 import Sampling, ops
    from borrowed_compute_b200.engine import StepEntry
    from borrowed_compute_b200.sampling import RowSampler

    batch = len(prompts)
    slots = [eng.acquire() for _ in range(batch)]
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(0, batch, prompts_a_step):   # prompts in steps of a few, to bound activation memory
        eng.step([StepEntry(s, p, want=()) for s, p in zip(slots[i:i + prompts_a_step], prompts[i:i + prompts_a_step])])
    b.record()
    sampler = RowSampler(eng.rt.device, batch)
    sampler.set_rows([Sampling()] * batch)
    steps_t = torch.zeros(batch, dtype=torch.int32, device=eng.rt.device)
    toks = [[int(t) for t in rng.integers(0, vocab, batch)] for _ in range(steps + warmup)]

    def one(i):
        scores = eng.step([StepEntry(s, (toks[i][j],), want=(0,)) for j, s in enumerate(slots)], borrow_scores=True)
        sampler.sample(scores, steps_t)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    prompt_ms = a.elapsed_time(b)
    before = ops.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = ClockSampler() if sample_clocks else None
    if clocks:
        clocks.__enter__()
        time.sleep(0.3)
    torch.cuda.synchronize()
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    stop.record()
    torch.cuda.synchronize()
    if clocks:
        time.sleep(0.2)
        clocks.__exit__()
    ms = start.elapsed_time(stop)
    cached = sum(len(p) for p in prompts) + batch * (warmup + steps / 2.0)     # positions the live requests hold, mid-run
    for s in slots:
        eng.release(s)
    eng.raise_on_kernel_error()
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1000.0), "cached_tokens": cached, "prompt_ms": prompt_ms,
            "clocks": clocks.summary() if clocks else None, "eager_launches": ops.launches - before}


def breakdown(eng, cfg, layers, batch, pk, rng):
    """Every kernel class of one decode step (``batch`` sequences after 2,048-token prompts)
    and of one 2,048-token prompt step, launch by launch, against its own bytes or operations."""
    from borrowed_compute_b200 import Sampling
    from borrowed_compute_b200.engine import StepEntry, StepProfile
    from borrowed_compute_b200.sampling import RowSampler
    import torch

    vocab = cfg["vocab_size"]
    slots = [eng.acquire() for _ in range(batch)]
    prompts = [[int(t) for t in rng.integers(0, vocab, PROMPT)] for _ in range(batch)]
    for i in range(0, batch, 8):
        eng.step([StepEntry(s, p, want=()) for s, p in zip(slots[i:i + 8], prompts[i:i + 8])])
    sampler = RowSampler(eng.rt.device, batch)
    sampler.set_rows([Sampling()] * batch)
    steps_t = torch.zeros(batch, dtype=torch.int32, device=eng.rt.device)

    def one():
        scores = eng.step([StepEntry(s, (int(rng.integers(0, vocab)),), want=(0,)) for s in slots])
        sampler.sample(scores, steps_t)

    reps = 5
    with StepProfile(eng) as warm:
        one()
    with StepProfile(eng) as prof:
        for _ in range(reps):
            one()
    decode = prof.classes(reps)
    for s in slots:
        eng.release(s)
    slot = eng.acquire()
    p = prompts[0]
    with StepProfile(eng) as warm:   # noqa: F841
        eng.step([StepEntry(slot, p, want=(PROMPT - 1,))])
    eng.rollback(slot, 0)
    with StepProfile(eng) as prof:
        for _ in range(3):
            eng.step([StepEntry(slot, p, want=(PROMPT - 1,))])
            eng.rollback(slot, 0)
    prefill = prof.classes(3)
    eng.release(slot)
    costs = class_costs(cfg, layers, batch, batch * (PROMPT + 3), PROMPT)
    out = {"decode": {}, "prefill": {}, "how": "eager steps, CUDA events around every launch (no overlap between launches): shares, not a step's time"}
    for cls, m in sorted(decode.items(), key=lambda kv: -kv[1]["us"]):
        row = {"us": round(m["us"], 1), "launches": round(m["launches"], 1)}
        if cls in costs["decode"]:
            gbs = costs["decode"][cls] / (m["us"] * 1e-6) / 1e9
            row.update({"bytes": int(costs["decode"][cls]), "gb_s": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 3)})
        out["decode"][cls] = row
    for cls, m in sorted(prefill.items(), key=lambda kv: -kv[1]["us"]):
        row = {"us": round(m["us"], 1), "launches": round(m["launches"], 1)}
        if cls in costs["prefill"]:
            kind, amount = costs["prefill"][cls]
            if kind == "flops":
                tf = amount / (m["us"] * 1e-6) / 1e12
                row.update({"flops": float(amount), "tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 3)})
            else:
                gbs = amount / (m["us"] * 1e-6) / 1e9
                row.update({"bytes": int(amount), "gb_s": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 3)})
        out["prefill"][cls] = row
    out["decode_sum_us"] = round(sum(m["us"] for m in decode.values()), 1)
    out["prefill_sum_us"] = round(sum(m["us"] for m in prefill.values()), 1)
    return out


def bench_tiny(rng) -> dict:
    """The two tiny workloads (float32): a batch of 3 prompts of 5 / 17 / 1 tokens and 8 greedy
    steps; a batch of 4 prompts of 1 / 9 / 33 / 70 tokens and 16 steps at temperature 0.8,
    top_p 0.9.  Through the entry point on the device, and through the plain C++ twin on the
    host (which recomputes the whole sequence every step): the twin's time is the CPU baseline,
    and its tokens must be the engine's."""
    import torch

    from borrowed_compute_b200 import Local, Sampling, twin
    from borrowed_compute_b200.weights import random_tensors

    out = {}
    for name, cfg, lengths, new, sampling in (("tiny_a", CONFIG_TINY_A, (5, 17, 1), 8, Sampling()),
                                              ("tiny_b", CONFIG_TINY_B, (1, 9, 33, 70), 16, Sampling(temperature=0.8, top_p=0.9, seed=1234567))):
        model = Local.random(cfg, seed=1, dtype="float32", max_tokens=1024, max_slots=4, max_seq=cfg["max_position_embeddings"])
        weights = {k: v.float().cpu().numpy() for k, v in random_tensors(model.engine.model.expected_tensors(), 1, torch.float32, "cuda").items()}
        host = twin.TwinLlama(cfg, weights)
        prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], n)] for n in lengths]
        model.generate(prompts, new, sampling, stop_ids=())                      # first-use set-up outside the timed call
        started = time.perf_counter()
        got, _ = model.generate(prompts, new, sampling, stop_ids=())
        engine_ms = 1000.0 * (time.perf_counter() - started)
        started = time.perf_counter()
        want = [host.generate(p, new, sampling.temperature, sampling.top_p, sampling.seed) for p in prompts]
        twin_ms = 1000.0 * (time.perf_counter() - started)
        if got != want:
            raise AssertionError(f"bench: {name}: the engine generated {got}, the plain C++ twin {want}")
        out[f"{name}_engine_ms"], out[f"{name}_cpu_twin_ms"] = round(engine_ms, 2), round(twin_ms, 2)
        del model
    free_device_memory()
    return out


def bench_13b(pk, rng) -> dict:
    """The Llama-2-13B shape: 16 prompts of unequal lengths (uniform in 64 .. 2,048, seeded)
    in ONE ragged prompt step, then 128 decode steps, device-timed."""
    from borrowed_compute_b200 import Local

    cfg, layers = CONFIG_13B, CONFIG_13B["num_hidden_layers"]
    lengths = [int(n) for n in rng.integers(64, 2049, 16)]
    steps, warmup = 128, 4
    max_tokens = sum(-(-(n + steps + warmup + 8) // 64) * 64 for n in lengths)
    model = Local.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_slots=16, max_seq=cfg["max_position_embeddings"])
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], n)] for n in lengths]
    r = timed_decode(model.engine, prompts, steps, warmup, rng, cfg["vocab_size"], prompts_a_step=16)
    need = decode_bytes(cfg, layers, 16, r["cached_tokens"])
    gbs = need / (r["ms_per_step"] / 1000.0) / 1e9
    flops = prefill_flops(cfg, layers, lengths)
    out = {"llama2_13b_mha_decode_b16": round(r["tok_s"], 1), "llama2_13b_mha_ms_per_step": round(r["ms_per_step"], 4),
           "llama2_13b_mha_bytes_per_step": int(need), "llama2_13b_mha_hbm_frac": round(gbs / pk["hbm_gbs"], 4),
           "llama2_13b_mha_prompt_tokens": sum(lengths), "llama2_13b_mha_prefill_tok_s": round(sum(lengths) / (r["prompt_ms"] / 1000.0), 1),
           "llama2_13b_mha_prefill_frac": round(flops / (r["prompt_ms"] / 1000.0) / (pk["bf16_tflops"] * 1e12), 4)}
    del model
    free_device_memory()
    return out


def bench_long(pk, rng, layers=0) -> dict:
    """The 8B shape with one sequence of 32,000 tokens (the context that Llama-3.1 is made
    for is 131,072): the prompt in ONE step, then 64 decode steps, device-timed.  At this
    length a decode step reads 4 GB of keys and values beside the 16 GB of weights, and the
    prompt's work is half attention."""
    from borrowed_compute_b200 import Local

    layers = layers or CONFIG_8B["num_hidden_layers"]
    cfg = dict(CONFIG_8B, max_position_embeddings=32768, num_hidden_layers=layers)
    length, steps, warmup = 32000, 64, 4
    model = Local.random(cfg, seed=0, dtype="bfloat16", max_tokens=32768, max_slots=1, max_seq=32768)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], length)]]
    r = timed_decode(model.engine, prompts, steps, warmup, rng, cfg["vocab_size"], prompts_a_step=1)
    need = decode_bytes(cfg, layers, 1, r["cached_tokens"])
    flops = prefill_flops(cfg, layers, [length])
    out = {"decode_b1_ctx32k_layers": layers, "decode_b1_ctx32k": round(r["tok_s"], 1), "decode_b1_ctx32k_ms_per_step": round(r["ms_per_step"], 4),
           "decode_b1_ctx32k_hbm_frac": round(need / (r["ms_per_step"] / 1000.0) / 1e9 / pk["hbm_gbs"], 4),
           "prefill_32k_tok_s": round(length / (r["prompt_ms"] / 1000.0), 1),
           "prefill_32k_frac": round(flops / (r["prompt_ms"] / 1000.0) / (pk["bf16_tflops"] * 1e12), 4)}
    del model
    free_device_memory()
    return out


def bench_3b(pk, rng) -> dict:
    """The Llama-3.2-3B shape (tied head): 64 prompts of 1,024 tokens, then 512 tokens each
    sampled at temperature 1.0, through the entry point (the sampler runs every step)."""
    from borrowed_compute_b200 import Local, Sampling

    cfg, layers = CONFIG_3B, CONFIG_3B["num_hidden_layers"]
    batch, prompt, new = 64, 1024, 512
    model = Local.random(cfg, seed=0, dtype="bfloat16", max_tokens=batch * (-(-(prompt + new + 8) // 64) * 64), max_slots=batch,
                         max_seq=prompt + new + 8)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], prompt)] for _ in range(batch)]
    model.generate(prompts[:2], 4, Sampling(temperature=1.0, seed=1), stop_ids=())      # first-use set-up outside the timed call
    out, stats = model.generate(prompts, new, Sampling(temperature=1.0, top_p=1.0, seed=7), stop_ids=())
    assert all(len(o) == new for o in out)
    tok_s = stats.decode_tokens_per_second
    ms = 1000.0 * batch / tok_s
    need = decode_bytes(cfg, layers, batch, batch * (prompt + new / 2.0))
    res = {"llama32_3b_sampled_e2e_b64": round(tok_s, 1), "llama32_3b_sampled_ms_per_step": round(ms, 4),
           "llama32_3b_sampled_bytes_per_step": int(need), "llama32_3b_sampled_hbm_frac": round(need / (ms / 1000.0) / 1e9 / pk["hbm_gbs"], 4),
           "llama32_3b_prefill_tok_s": round(batch * prompt / (stats.first_token_ms / 1000.0), 1)}
    del model
    free_device_memory()
    return res


def run_ours(args) -> dict:
    import numpy as np
    import torch

    from borrowed_compute_b200 import Local, Sampling, ops
    from borrowed_compute_b200.engine import StepEntry
    from borrowed_compute_b200.engine import engine as engine_module

    global PROMPT
    PROMPT = args.prompt
    cfg = dict(CONFIG_8B)
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or full_layers
    layers = cfg["num_hidden_layers"]
    vocab = cfg["vocab_size"]
    pk = peaks()
    rng = np.random.default_rng(0)
    biggest = max(args.batch, 64 if not args.no_points else args.batch)
    new_tokens = max(args.warmup, E2E_SETTLE_PASSES) + args.steps + 8
    max_tokens = biggest * (-(-(PROMPT + new_tokens + 64) // 64) * 64)
    model = Local.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_slots=biggest, max_seq=CONTEXT)
    eng = model.engine
    torch.cuda.synchronize()

    def prompts(batch):
        return [[int(t) for t in rng.integers(0, vocab, PROMPT)] for _ in range(batch)]

    # --- the headline: decode at the requested batch, timed on the device
    main = timed_decode(eng, prompts(args.batch), args.steps, args.warmup, rng, vocab, sample_clocks=True)
    # kernels a step: count them on one eager (uncaptured) step
    eng.use_graphs = False
    s = eng.acquire()
    eng.step([StepEntry(s, [1, 2, 3], want=())])
    before = ops.launches
    eng.step([StepEntry(s, (5,), want=(0,))])
    launches_per_step = ops.launches - before + 2   # + the two kernels of greedy sampling
    eng.release(s)
    eng.use_graphs = True

    need = decode_bytes(cfg, layers, args.batch, main["cached_tokens"])
    achieved = need / (main["ms_per_step"] / 1000.0) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(need), "peak_source": pk["source"]}

    # --- prefill of 2,048 tokens (one prompt, scores at its last token)
    slot = eng.acquire()
    p = prompts(1)[0]
    for _ in range(2):
        eng.step([StepEntry(slot, p, want=(PROMPT - 1,))])
        eng.rollback(slot, 0)
    torch.cuda.synchronize()
    times = []
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step([StepEntry(slot, p, want=(PROMPT - 1,))])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        eng.rollback(slot, 0)
    eng.release(slot)
    pms = min(times)
    flops = prefill_flops(cfg, layers, [PROMPT])
    prefill = {"value": round(PROMPT / (pms / 1000.0), 1), "tokens": PROMPT, "ms": round(pms, 3),
               "frac": round(flops / (pms / 1000.0) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(flops / (pms / 1000.0) / 1e12, 1)}
    if "bf16_tflops_sustained" in pk:   # what the same library product holds for seconds under the power cap, beside the burst figure above
        prefill["frac_of_sustained"] = round(flops / (pms / 1000.0) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    # --- end to end through the Python entry point: host ids in, host ids out, every step.
    # Passes that are not timed, then exactly K passes, timed on the host from the arrival of one
    # pass's ids to that of the K-th pass after it.  The untimed passes are W, but at least 24:
    # after the prompt burst (which runs into the power cap) the part takes 11 to 19 decode steps
    # to raise its clocks again, and a generation goes on straight from its prompt, so a timed
    # region that began after 3 passes would time that recovery, not decoding.  (The device-timed
    # figure above is taken after a host pause of 0.3 s, during which the clocks recover at once.)
    def end_to_end(batch, steps, warmup):
        warmup = max(warmup, E2E_SETTLE_PASSES)
        ps = prompts(batch)
        traffic = engine_module.TRAFFIC
        arrived = []
        seen = {"h2d": 0, "d2h": 0}

        def on_token(i, tok):
            if i == 0:
                arrived.append(time.perf_counter())
                if len(arrived) == warmup + 1:
                    seen["h2d"], seen["d2h"] = traffic["h2d_decode"], traffic["d2h_decode"]

        out, stats = model.generate(ps, warmup + steps + 1, Sampling(), on_token=on_token, stop_ids=())
        seconds = arrived[warmup + steps] - arrived[warmup]
        per_step = float(steps)
        return {"prompts": ps, "out": out, "stats": stats, "tok_s": batch * steps / seconds, "ms_per_step": 1000.0 * seconds / steps, "warmup": warmup,
                "h2d": (traffic["h2d_decode"] - seen["h2d"]) / per_step, "d2h": (traffic["d2h_decode"] - seen["d2h"]) / per_step}

    r = end_to_end(args.batch, args.steps, args.warmup)
    ps, out, stats = r["prompts"], r["out"], r["stats"]
    e2e = {"value": round(r["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": int(round(r["h2d"])),
           "d2h_bytes_per_step": int(round(r["d2h"])), "ms_per_step": round(r["ms_per_step"], 4), "generated": stats.generated,
           "passes": stats.passes, "untimed_passes": r["warmup"], "first_token_ms": round(stats.first_token_ms, 1),
           "of_device_timed": round(r["tok_s"] / main["tok_s"], 4)}
    # --- the check: the same prompts stepped launch by launch (no captured graph, no step begun ahead) give the same tokens
    eng.use_graphs = False
    plain_out, _ = model.generate(ps, r["warmup"] + args.steps + 1, Sampling(), stop_ids=())
    eng.use_graphs = True
    if plain_out != out:
        bad = next(i for i, (x, y) in enumerate(zip(out, plain_out)) if x != y)
        raise AssertionError(f"bench: sequence {bad} generated {out[bad][:8]}... through captured steps and {plain_out[bad][:8]}... step by step")
    if len({tuple(o) for o in out}) < len(out) or any(not 0 <= t < vocab for o in out for t in o):
        raise AssertionError("bench: the generated sequences are not distinct sequences of token ids")

    classes = None if args.no_breakdown else breakdown(eng, cfg, layers, args.batch, pk, rng)

    points = {}
    if not args.no_points:
        for b in (1, 64):
            r = timed_decode(eng, prompts(b), max(16, args.steps // 2), max(3, args.warmup // 2), rng, vocab)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            need_b = decode_bytes(cfg, layers, b, r["cached_tokens"])
            points[f"decode_b{b}_hbm_frac"] = round(need_b / (r["ms_per_step"] / 1000.0) / 1e9 / pk["hbm_gbs"], 4)
            e = end_to_end(b, max(16, args.steps // 2), max(3, args.warmup // 2))
            points[f"e2e_b{b}"] = round(e["tok_s"], 1)
            points[f"e2e_b{b}_of_device_timed"] = round(e["tok_s"] / r["tok_s"], 4)
    del model, eng
    free_device_memory()
    if not args.no_points and not args.layers:
        points.update(bench_long(pk, rng))
        points.update(bench_13b(pk, rng))
        points.update(bench_3b(pk, rng))
        points.update(bench_tiny(rng))

    config = {"model": "llama-3.1-8b-shape", "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
              "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
              "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
              "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single-gpu", "l2": "inputs larger than L2 (16 GB of weights a step)"}
    line = {
        "metric": "decode tokens/s (Llama-3.1-8B shape, bf16, batch %d, 2,048-token prompts)" % args.batch,
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random N(0,0.02) weights", "config": config,
        "clocks": main["clocks"], "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "launches_per_step": launches_per_step,
        "prefill": prefill, "roofline": roofline, "points": points, "checked": True, "impl": "ours",
    }
    if classes is not None:
        line["classes"] = classes
    return line


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt tokens before the timed decode steps")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64 and the two other shapes")
    ap.add_argument("--no-breakdown", action="store_true", help="skip the per-class timing of one decode and one prompt step")
    ap.add_argument("--point", default="", choices=["", "long", "13b", "3b", "tiny"],
                    help="run one of the further workloads alone and print its figures (not the contract's line)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust workspace (no setup.py or pyproject) "
                          "and no Rust toolchain is installed: it can be neither pip-installed nor built here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported (this library does not use several GPUs)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.point:
        import numpy as np

        rng = np.random.default_rng(0)
        one = {"long": lambda: bench_long(peaks(), rng, args.layers), "13b": lambda: bench_13b(peaks(), rng), "3b": lambda: bench_3b(peaks(), rng),
               "tiny": lambda: bench_tiny(rng)}[args.point]
        print(json.dumps({"point": args.point, **one()}))
        return 0
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
