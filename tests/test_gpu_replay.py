"""bin/trace_run, as a user runs it: the same requests replayed whole, with the last 32
tokens one by one, and in batches of unequal lengths one after another (so slots are used
again), in float32 and bfloat16, all compared with the plain implementation."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama
from conftest import ROOT, TINY, seeded_tokens, tolerance

pytestmark = pytest.mark.gpu

TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(folder, dtype, out_dir, steps, max_tokens):
    """Feeds the steps one at a time, waiting for each `done` line as the protocol says."""
    proc = subprocess.Popen([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


def scores_of(out_dir, step, vocab):
    return np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)


def requests_for(name):
    vocab = TINY[name]["vocab_size"]
    lengths = {"A": [40, 7, 100, 65], "B": [70, 33, 150, 64]}[name]
    return {f"r{i}": seeded_tokens(300 + i, n, vocab) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_three_ways_of_cutting(model_folders, tmp_path, name, dtype):
    folder, cfg, weights = model_folders(name, dtype)
    vocab = cfg["vocab_size"]
    reqs = requests_for(name)
    ref = {rid: plain_llama.logits(cfg, weights, toks) for rid, toks in reqs.items()}
    steps, expect = [], {}     # expect[step] = list of (request, positions)
    n = 0
    # 1. each request alone and whole
    for rid, toks in reqs.items():
        steps.append({"step": n, "entries": [{"id": rid + "w", "tokens": toks, "want": list(range(len(toks)))}], "end": [rid + "w"]})
        expect[n] = [(rid, list(range(len(toks))))]
        n += 1
    # 2. all but the last 32 tokens at once, then the last 32 one by one
    for rid, toks in reqs.items():
        if len(toks) <= 32:
            continue
        cut = len(toks) - 32
        steps.append({"step": n, "entries": [{"id": rid + "d", "tokens": toks[:cut], "want": [cut - 1]}], "end": []})
        expect[n] = [(rid, [cut - 1])]
        n += 1
        for i in range(cut, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid + "d", "tokens": [toks[i]], "want": [0]}], "end": [rid + "d"] if i == len(toks) - 1 else []})
            expect[n] = [(rid, [i])]
            n += 1
    # 3. two batches of unequal lengths, one after the other; shorter requests end earlier
    for batch in (["r0", "r1", "r2"], ["r3", "r1", "r0"]):
        tail = 5
        live = [(rid, reqs[rid]) for rid in batch]
        steps.append({"step": n, "end": [], "entries": [{"id": rid + "b", "tokens": t[:max(1, len(t) - tail)], "want": [max(1, len(t) - tail) - 1]}
                                                        for rid, t in live]})
        expect[n] = [(rid, [max(1, len(t) - tail) - 1]) for rid, t in live]
        n += 1
        at = {rid: max(1, len(t) - tail) for rid, t in live}
        # the request with index 1 stops two tokens early: it leaves the batch before the others
        stop_at = {rid: len(t) - (2 if j == 1 else 0) for j, (rid, t) in enumerate(live)}
        while any(at[rid] < stop_at[rid] for rid, _ in live):
            going = [(rid, t) for rid, t in live if at[rid] < stop_at[rid]]
            ends = [rid + "b" for rid, t in going if at[rid] + 1 == stop_at[rid]]
            steps.append({"step": n, "entries": [{"id": rid + "b", "tokens": [t[at[rid]]], "want": [0]} for rid, t in going], "end": ends})
            expect[n] = [(rid, [at[rid]]) for rid, t in going]
            for rid, _ in going:
                at[rid] += 1
            n += 1
    # the largest demand at any time: the biggest batch, each request rounded up to 64
    need = max(sum(-(-len(reqs[r]) // 64) * 64 for r in b) for b in (["r0", "r1", "r2"], ["r3", "r1", "r0"]))
    out_dir = str(tmp_path / "out")
    replay(folder, dtype, out_dir, steps, need)
    for step, wanted in expect.items():
        got = scores_of(out_dir, step, vocab)
        want = np.concatenate([ref[rid][pos] for rid, pos in wanted])
        assert got.shape == want.shape, f"step {step}"
        err = float(np.abs(got - want).max())
        assert err <= tolerance(dtype, want), f"step {step} ({wanted}): error {err:.3e}"


def test_steps_without_wants_write_nothing(model_folders, tmp_path):
    folder, cfg, _ = model_folders("A", "float32")
    out_dir = str(tmp_path / "out")
    replay(folder, "float32", out_dir, [
        {"step": 0, "entries": [{"id": "x", "tokens": [1, 2, 3], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "x", "tokens": [4], "want": [0]}], "end": ["x"]},
        {"step": 2, "entries": [], "end": []},
    ], 64)
    assert sorted(os.listdir(out_dir)) == ["1.f32"]
    assert scores_of(out_dir, 1, cfg["vocab_size"]).shape == (1, cfg["vocab_size"])
