"""Decode and prefill throughput of the Llama-3.1-8B shape on one B200, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  ``value`` is decoded
tokens a second timed on the device (CUDA events around K steps, after W warm-up steps);
``e2e`` is the same through the Python entry point (host token ids in, host token ids out
every step); ``prefill`` is one 2,048-token prompt; ``roofline`` sets the decode step's
mandatory bytes (every weight once, the live requests' cache once) against the measured
copy bandwidth; ``points`` adds batch 1 and 64.  Every decode step streams all weights
(16 GB), far more than the 126 MB L2, so nothing is flushed between iterations.

The reference (Harshil089/Borrowed-Compute) is a Rust workspace; no Rust toolchain exists
here, so ``--impl reference`` reports itself unavailable.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Llama-3.1-8B shape.
CONFIG_8B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}
CONTEXT = 8192
PROMPT = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


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


def model_numbers(cfg: dict, layers: int):
    E, H, G, D, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                        cfg["intermediate_size"], cfg["vocab_size"])
    layer_params = E * (H + 2 * G) * D + H * D * E + 3 * E * F
    return {"layer_params": layer_params, "head_params": V * E, "norm_params": (2 * layers + 1) * E,
            "kv_bytes_per_token": layers * 2 * G * D * 2, "E": E, "H": H, "D": D, "V": V}


def decode_bytes(cfg, layers, batch, context) -> float:
    n = model_numbers(cfg, layers)
    weights = 2.0 * (layers * n["layer_params"] + n["head_params"]) + 4.0 * n["norm_params"] + 2.0 * batch * n["E"]
    return weights + float(batch) * context * n["kv_bytes_per_token"]


def prefill_flops(cfg, layers, tokens) -> float:
    n = model_numbers(cfg, layers)
    linear = 2.0 * tokens * layers * n["layer_params"]
    attention = layers * 2.0 * 2.0 * n["H"] * n["D"] * tokens * (tokens + 1) / 2.0
    return linear + attention + 2.0 * n["head_params"]


def run_ours(args) -> dict:
    import numpy as np
    import torch

    from borrowed_compute_b200 import Local, Sampling, ops
    from borrowed_compute_b200.engine import StepEntry
    from borrowed_compute_b200.sampling import RowSampler

    global PROMPT
    PROMPT = args.prompt
    cfg = dict(CONFIG_8B)
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or full_layers
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    rng = np.random.default_rng(0)
    biggest = max(args.batch, 64 if not args.no_points else args.batch)
    new_tokens = args.warmup + args.steps + 8
    max_tokens = biggest * (-(-(PROMPT + new_tokens + 64) // 64) * 64)
    model = Local.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_slots=biggest, max_seq=CONTEXT)
    eng = model.engine
    torch.cuda.synchronize()

    def prompts(batch):
        return [[int(t) for t in rng.integers(0, cfg["vocab_size"], PROMPT)] for _ in range(batch)]

    def timed_decode(batch, steps, warmup, sample_clocks=False):
        """Device time of `steps` decode steps of `batch` sequences after 2,048-token prompts."""
        slots = [eng.acquire() for _ in range(batch)]
        ps = prompts(batch)
        for i in range(0, batch, 8):   # prompts in steps of at most 8, to bound activation memory
            eng.step([StepEntry(s, p, want=()) for s, p in zip(slots[i:i + 8], ps[i:i + 8])])
        sampler = RowSampler(eng.rt.device, batch)
        sampler.set_rows([Sampling()] * batch)
        steps_t = torch.zeros(batch, dtype=torch.int32, device=eng.rt.device)
        toks = [[int(t) for t in rng.integers(0, cfg["vocab_size"], batch)] for _ in range(steps + warmup)]

        def one(i):
            scores = eng.step([StepEntry(s, (toks[i][j],), want=(0,)) for j, s in enumerate(slots)])
            sampler.sample(scores, steps_t)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
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
        context = PROMPT + warmup + steps / 2.0
        for s in slots:
            eng.release(s)
        return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1000.0), "context": context,
                "clocks": clocks.summary() if clocks else None, "eager_launches": ops.launches - before}

    # --- the headline: decode at the requested batch
    main = timed_decode(args.batch, args.steps, args.warmup, sample_clocks=True)
    # kernels a step: count them on one eager (uncaptured) step
    eng.use_graphs = False
    s = eng.acquire()
    eng.step([StepEntry(s, [1, 2, 3], want=())])
    before = ops.launches
    eng.step([StepEntry(s, (5,), want=(0,))])
    launches_per_step = ops.launches - before + 2   # + the two kernels of greedy sampling
    eng.release(s)
    eng.use_graphs = True

    need = decode_bytes(cfg, layers, args.batch, main["context"])
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
    flops = prefill_flops(cfg, layers, PROMPT)
    prefill = {"value": round(PROMPT / (pms / 1000.0), 1), "tokens": PROMPT, "ms": round(pms, 3),
               "frac": round(flops / (pms / 1000.0) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(flops / (pms / 1000.0) / 1e12, 1)}

    # --- end to end through the Python entry point: host ids in, host ids out, every step
    e2e_steps = args.steps
    out, stats = model.generate(prompts(args.batch), e2e_steps + 1, Sampling(), stop_ids=())
    e2e_tok_s = stats.decode_tokens_per_second
    rows = eng._bucket(args.batch)
    e2e = {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": (7 * rows + 1) * 4,
           "d2h_bytes_per_step": args.batch * 4, "generated": stats.generated, "passes": stats.passes,
           "first_token_ms": round(stats.first_token_ms, 1)}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            r = timed_decode(b, max(16, args.steps // 2), max(3, args.warmup // 2))
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            need_b = decode_bytes(cfg, layers, b, r["context"])
            points[f"decode_b{b}_hbm_frac"] = round(need_b / (r["ms_per_step"] / 1000.0) / 1e9 / pk["hbm_gbs"], 4)

    config = {"model": "llama-3.1-8b-shape", "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
              "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
              "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
              "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single-gpu", "l2": "inputs larger than L2 (16 GB of weights a step)"}
    return {
        "metric": "decode tokens/s (Llama-3.1-8B shape, bf16, batch %d, 2,048-token prompts)" % args.batch,
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random N(0,0.02) weights", "config": config,
        "clocks": main["clocks"], "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "launches_per_step": launches_per_step,
        "prefill": prefill, "roofline": roofline, "points": points, "impl": "ours",
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt tokens before the timed decode steps")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
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
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
