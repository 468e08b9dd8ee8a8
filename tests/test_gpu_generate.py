"""Generation through the Python entry point and the command line, against the plain
implementation's loop: greedy and sampled, batches of unequal prompts, stop tokens."""

from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama
from conftest import ROOT, TINY, seeded_tokens, tolerance

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def locals_(model_folders):
    from borrowed_compute_b200 import Local

    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            folder, cfg, weights = model_folders(name, dtype)
            made[(name, dtype)] = (Local.load(folder, dtype=dtype, max_tokens=1024, max_slots=4), cfg, weights, folder)
        return made[(name, dtype)]

    return get


def greedy_within_rounding(cfg, weights, prompt, out, dtype):
    """Every generated token is a largest score of the plain implementation at its place,
    within the tolerance of the path: the greedy choice, up to rounding between near ties."""
    seq = list(prompt) + list(out)
    ref = plain_llama.logits(cfg, weights, seq[:-1]) if len(seq) > 1 else None
    for i, tok in enumerate(out):
        row = ref[len(prompt) - 1 + i]
        assert row.max() - row[tok] <= 2 * tolerance(dtype, row), f"token {i} ({tok}) is not a greedy choice"


def test_greedy_batch_of_three_in_float32(locals_):
    """Tiny A's workload: prompts of 5, 17 and 1 tokens, eight greedy steps."""
    from borrowed_compute_b200 import Sampling

    model, cfg, weights, _ = locals_("A", "float32")
    prompts = [seeded_tokens(20 + i, n, cfg["vocab_size"]) for i, n in enumerate([5, 17, 1])]
    out, stats = model.generate(prompts, 8, Sampling(), stop_ids=())
    assert out == [plain_llama.generate(cfg, weights, p, 8) for p in prompts]
    assert stats.prompt_tokens == 23 and stats.generated == 24 and stats.passes == 7 and stats.first_token_ms > 0
    assert model.engine.cache.slots.live() == []


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_in_bfloat16(locals_, name):
    from borrowed_compute_b200 import Sampling

    model, cfg, weights, _ = locals_(name, "bfloat16")
    prompts = [seeded_tokens(30 + i, n, cfg["vocab_size"]) for i, n in enumerate([9, 33, 2])]
    out, _ = model.generate(prompts, 12, Sampling(), stop_ids=())
    for p, o in zip(prompts, out):
        assert len(o) == 12
        greedy_within_rounding(cfg, weights, p, o, "bfloat16")


def test_sampled_batch_of_four_in_float32(locals_):
    """Tiny B's workload: prompts of 1, 9, 33 and 70 tokens, sixteen steps at temperature
    0.8, top_p 0.9, a fixed seed; and the same requests alone draw the same tokens."""
    from borrowed_compute_b200 import Sampling

    model, cfg, weights, _ = locals_("B", "float32")
    prompts = [seeded_tokens(40 + i, n, cfg["vocab_size"]) for i, n in enumerate([1, 9, 33, 70])]
    s = Sampling(temperature=0.8, top_p=0.9, seed=1234567)
    out, _ = model.generate(prompts, 16, s, stop_ids=())
    want = [plain_llama.generate(cfg, weights, p, 16, temperature=0.8, top_p=0.9, seed=1234567) for p in prompts]
    assert out == want
    assert len({tuple(o) for o in out}) == 4
    for p, o in zip(prompts, out):
        alone, _ = model.generate(p, 16, s, stop_ids=())
        assert alone == o, "a sequence must sample the same alone as in a batch"
    other, _ = model.generate(prompts, 16, Sampling(temperature=0.8, top_p=0.9, seed=7), stop_ids=())
    assert other != out


def test_stop_tokens_and_more_requests_than_slots(locals_):
    from borrowed_compute_b200 import Sampling

    model, cfg, weights, _ = locals_("B", "float32")
    prompts = [seeded_tokens(60 + i, 3 + 5 * i, cfg["vocab_size"]) for i in range(7)]
    free = [plain_llama.generate(cfg, weights, p, 10) for p in prompts]
    stops = {free[0][3], free[4][0]}
    want = [plain_llama.generate(cfg, weights, p, 10, stops=stops) for p in prompts]
    assert any(len(w) < 10 for w in want)
    out, stats = model.generate(prompts, 10, Sampling(), stop_ids=sorted(stops), max_batch=3)   # three batches: 3 + 3 + 1
    assert out == want and model.engine.cache.slots.live() == []
    default, _ = model.generate(prompts[:2], 4, Sampling())                                       # the model's own eos ids apply
    assert all(t not in (7, 300) for o in default for t in o)


def test_scores_follow_the_reference_contract(locals_):
    """crates/bc-infer/src/model.rs:520-534: a prompt then a step equals the whole sequence;
    going back and running again gives the same scores; skipping ahead is an error."""
    model, cfg, weights, _ = locals_("A", "float32")
    tokens = seeded_tokens(70, 12, cfg["vocab_size"])
    ref = plain_llama.logits(cfg, weights, tokens)
    model.reset()
    first = model.scores(tokens[:8], 0).numpy()
    step = model.scores(tokens[8:], 8).numpy()
    assert np.abs(np.concatenate([first, step]) - ref).max() <= tolerance("float32", ref)
    again = model.scores(tokens[8:], 8).numpy()
    assert np.array_equal(step, again)
    with pytest.raises(ValueError, match="skips past"):
        model.scores([1], 40)
    model.reset()


def test_command_line(locals_, tmp_path):
    _, cfg, weights, folder = locals_("A", "float32")
    prompts = [[5, 17, 3], [9]]
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bc-infer"), "generate", folder, "5,17,3;9", "--max-tokens", "6",
                          "--dtype", "float32", "--stop-ids", ""], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    got = [[int(t) for t in line.split(",")] for line in res.stdout.strip().splitlines()]
    assert got == [plain_llama.generate(cfg, weights, p, 6) for p in prompts]
    assert "prompt tokens, first token after" in res.stderr and "tokens/s" in res.stderr


def test_command_line_options_and_generation_config(locals_, tmp_path):
    """--max-seq, --stats and --include-stop; stop ids from generation_config.json; load progress."""
    import json
    import shutil

    from borrowed_compute_b200 import Local

    _, cfg, weights, folder = locals_("A", "float32")
    free = plain_llama.generate(cfg, weights, [5, 17, 3], 6)
    mine = str(tmp_path / "with_generation_config")
    shutil.copytree(folder, mine)
    with open(os.path.join(mine, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [free[3]]}, f)
    seen = []
    model = Local.load(mine, dtype="float32", max_tokens=256, progress=lambda done, total: seen.append((done, total)))
    assert free[3] in model.stop_ids and cfg["eos_token_id"] in model.stop_ids
    assert seen and seen[-1][0] == seen[-1][1] == len(seen)
    cut = free[:free.index(free[3])]
    assert model.generate([5, 17, 3], 6)[0] == cut
    assert model.generate([5, 17, 3], 6, include_stop=True)[0] == cut + [free[3]]
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bc-infer"), "generate", mine, "5,17,3", "--max-tokens", "6", "--dtype", "float32",
                          "--max-seq", "64", "--stats", "--include-stop"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    lines = res.stdout.strip().splitlines()
    assert [int(t) for t in lines[0].split(",")] == cut + [free[3]]
    stats = json.loads(lines[1])
    assert stats["prompt_tokens"] == 3 and stats["generated"] == len(cut) + 1 and stats["total_ms"] >= stats["first_token_ms"] > 0
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bc-infer"), "generate", mine, "5,17,3", "--max-tokens", "6", "--max-seq", "5"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode != 0 and "--max-seq" in res.stderr


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_engine_and_the_plain_cxx_twin_generate_the_same(locals_, name):
    """The third restatement of the formulas, in plain C++ on the host, against the engine in
    float32: the same tokens, greedy and sampled."""
    from borrowed_compute_b200 import Sampling, twin

    model, cfg, weights, _ = locals_(name, "float32")
    host = twin.TwinLlama(cfg, weights)
    prompts = [seeded_tokens(80 + i, n, cfg["vocab_size"]) for i, n in enumerate([7, 1, 40])]
    got, _ = model.generate(prompts, 10, Sampling(), stop_ids=())
    assert got == [host.generate(p, 10) for p in prompts]
    s = Sampling(temperature=0.9, top_p=0.85, seed=42)
    got, _ = model.generate(prompts, 10, s, stop_ids=())
    assert got == [host.generate(p, 10, 0.9, 0.85, 42) for p in prompts]
    scores = model.scores(prompts[2], 0).numpy()
    model.reset()
    ref = host.logits(prompts[2])
    assert np.abs(scores - ref).max() <= tolerance("float32", ref)
