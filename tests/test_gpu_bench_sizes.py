"""The benchmark's own model and sizes under test: the Llama-3.1-8B shape that bench.py
times (32 layers, hidden 4,096, a vocabulary of 128,256, prompts of 2,048 tokens), cut
every way the small configurations are cut.  The reference tests whole against cut on its
full path and past the edge of an attention tile and of the first cache allocation
(crates/bc-infer/src/model.rs:509-536, 613-674); here the same is asked at the sizes whose
numbers are reported.

In float32 every way of cutting the work gives the same bits.  The bfloat16 engine, through
its captured decode steps, is held to the float32 engine over the same (bfloat16-rounded)
weights within the suite's bound for deep models (conftest.deep_bf16_bounds: rounding noise
grows with the root of the depth); the float32 engine is held to the plain
implementation at the full vocabulary on two layers (thirty-two in float64 on the host are
out of reach).  Weights are the random ones bench.py draws.
"""

from __future__ import annotations

import gc

import numpy as np
import pytest

import plain_llama
from bench import CONFIG_8B
from conftest import F32_TOL, assert_deep_bf16

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

PROMPT, TAIL = 2048, 32
VOCAB = CONFIG_8B["vocab_size"]


def tokens(seed, n):
    return [int(t) for t in np.random.default_rng(seed).integers(0, VOCAB, n)]


REQ_A, REQ_B, REQ_C = tokens(1, PROMPT + TAIL), tokens(2, 700), tokens(3, 150)
TAILS = {"A": TAIL, "B": 20, "C": 10}     # tokens of each request that are fed one by one


@pytest.fixture(scope="module")
def engines():
    """The float32 and the bfloat16 engine of the full shape over the same stored values."""
    from borrowed_compute_b200 import Engine

    if torch.cuda.get_device_properties(0).total_memory < 100e9:
        pytest.skip("the full Llama-3.1-8B shape in float32 and bfloat16 needs about 60 GB")
    made = {}
    for dtype in ("float32", "bfloat16"):
        made[dtype] = Engine.from_random(CONFIG_8B, 0, dtype=dtype, stored_dtype="bfloat16", max_tokens=8192, max_slots=64, max_seq=4096)
    yield made
    made.clear()
    gc.collect()
    torch.cuda.empty_cache()


def run_cuts(eng):
    """Request A's last 32 rows of scores, whole, with its last 32 tokens one by one, and in
    a batch of three unequal requests run twice through the same slots; B's and C's rows from
    the batch and alone."""
    from borrowed_compute_b200 import StepEntry

    last = tuple(range(PROMPT, PROMPT + TAIL))
    out = {}
    s = eng.acquire()
    out["whole"] = eng.step([StepEntry(s, REQ_A, want=last)]).cpu().numpy()
    eng.release(s)
    s = eng.acquire()
    eng.step([StepEntry(s, REQ_A[:PROMPT], want=())])
    out["one by one"] = np.concatenate([eng.step([StepEntry(s, [t], want=(0,))]).cpu().numpy() for t in REQ_A[PROMPT:]])
    eng.release(s)
    for name, req in (("B alone", REQ_B), ("C alone", REQ_C)):
        s = eng.acquire()
        out[name] = eng.step([StepEntry(s, req, want=tuple(range(len(req) - TAILS[name[0]], len(req))))]).cpu().numpy()
        eng.release(s)
    for turn in ("batch", "batch again"):
        slots = {"A": eng.acquire(), "B": eng.acquire(), "C": eng.acquire()}
        reqs = {"A": REQ_A, "B": REQ_B, "C": REQ_C}
        fed = {k: len(reqs[k]) - TAILS[k] for k in reqs}      # C ends after ten more tokens, B after twenty, A after thirty-two
        eng.step([StepEntry(slots[k], reqs[k][:fed[k]], want=()) for k in ("C", "A", "B")])
        got = {k: [] for k in reqs}
        live = ["C", "A", "B"]
        while live:
            rows = eng.step([StepEntry(slots[k], [reqs[k][fed[k]]], want=(0,)) for k in live]).cpu().numpy()
            for i, k in enumerate(live):
                got[k].append(rows[i:i + 1])
                fed[k] += 1
            for k in list(live):
                if fed[k] == len(reqs[k]):
                    eng.release(slots[k])
                    live.remove(k)
        out[turn] = {k: np.concatenate(v) for k, v in got.items()}
    eng.cache.slots.check()
    assert eng.cache.slots.live() == []
    return out


def test_the_8b_shape_under_every_cut(engines):
    f32 = run_cuts(engines["float32"])
    ref = f32["whole"]
    assert np.isfinite(ref).all() and float(np.abs(ref).max()) > 1.0, "scores of a model that computes something"
    assert len({int(r.argmax()) for r in ref}) > 8, "rows differ"
    # float32: the same bits under every cut, in every batch, in slots used again
    assert np.array_equal(f32["one by one"], ref), "last 32 tokens one by one"
    for turn in ("batch", "batch again"):
        assert np.array_equal(f32[turn]["A"], ref), turn
        assert np.array_equal(f32[turn]["B"], f32["B alone"]) and np.array_equal(f32[turn]["C"], f32["C alone"]), turn
    # bfloat16 (captured decode steps; sizes 1, 2, 4): within the bound of the float32 engine over the same weights
    b16 = run_cuts(engines["bfloat16"])
    assert sorted(rows for rows, _ in engines["bfloat16"]._graphs) == [1, 2, 4]
    layers, worst = CONFIG_8B["num_hidden_layers"], 0.0
    for name, got, want in [("whole", b16["whole"], ref), ("one by one", b16["one by one"], ref), ("B alone", b16["B alone"], f32["B alone"]),
                            ("C alone", b16["C alone"], f32["C alone"])] + \
            [(f"{turn} {k}", b16[turn][k], {"A": ref, "B": f32["B alone"], "C": f32["C alone"]}[k]) for turn in ("batch", "batch again") for k in "ABC"]:
        worst = max(worst, assert_deep_bf16(got, want, layers, f"bfloat16 {name}"))
    # a launch repeated gives the same bits in bfloat16 too
    assert np.array_equal(b16["batch"]["A"], b16["batch again"]["A"])
    print(f"8B shape: scores of spread {ref.std():.3f}, the worst bfloat16 row differs by {worst:.4f} rms")


def test_a_decode_step_of_64_sequences(engines):
    """The captured step of 64 rows (the product's 64-token tile, 64 slots' page tables), with
    prompts of unequal lengths, against the float32 engine."""
    from borrowed_compute_b200 import StepEntry

    r = np.random.default_rng(9)
    lengths = [int(n) for n in r.integers(5, 120, 64)]
    prompts = [tokens(100 + i, n) for i, n in enumerate(lengths)]
    nxt = [tokens(200 + i, 3) for i in range(64)]
    res = {}
    for dtype, eng in engines.items():
        slots = [eng.acquire() for _ in range(64)]
        for i in range(0, 64, 16):
            eng.step([StepEntry(s, p, want=()) for s, p in zip(slots[i:i + 16], prompts[i:i + 16])])
        res[dtype] = [eng.step([StepEntry(s, [nxt[i][k]], want=(0,)) for i, s in enumerate(slots)]).cpu().numpy() for k in range(3)]
        for s in slots:
            eng.release(s)
    assert 64 in [rows for rows, _ in engines["bfloat16"]._graphs]
    for k in range(3):
        want, got = res["float32"][k], res["bfloat16"][k]
        assert got.shape == (64, VOCAB)
        assert_deep_bf16(got, want, CONFIG_8B["num_hidden_layers"], f"step {k}")
    # every sequence alone gives the float32 batch's bits
    eng = engines["float32"]
    for i in (0, 31, 63):
        s = eng.acquire()
        eng.step([StepEntry(s, prompts[i], want=())])
        alone = eng.step([StepEntry(s, [nxt[i][0]], want=(0,))]).cpu().numpy()
        eng.release(s)
        assert np.array_equal(alone[0], res["float32"][0][i])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_full_vocabulary_against_the_plain_implementation(dtype):
    """Two layers of the 8B shape with all 128,256 columns of the head, a short prompt then
    single tokens, against the plain implementation in float64 on the same stored values."""
    from borrowed_compute_b200 import Engine, StepEntry
    from borrowed_compute_b200.weights import random_tensors

    cfg = dict(CONFIG_8B, num_hidden_layers=2)
    eng = Engine.from_random(cfg, 3, dtype=dtype, stored_dtype="bfloat16", max_tokens=256, max_slots=2)
    drawn = random_tensors(eng.model.expected_tensors(), 3, torch.bfloat16, "cuda")
    weights = {k: v.float().cpu().numpy() for k, v in drawn.items()}
    del drawn
    req = tokens(5, 24)
    ref = plain_llama.logits(cfg, weights, req)
    del weights
    s = eng.acquire()
    got = [eng.step([StepEntry(s, req[:20], want=tuple(range(20)))]).cpu().numpy()]
    got += [eng.step([StepEntry(s, [t], want=(0,))]).cpu().numpy() for t in req[20:]]
    eng.release(s)
    got = np.concatenate(got)
    if dtype == "float32":
        assert np.abs(got - ref).max() <= F32_TOL * (1.0 + np.abs(ref).max())
    else:
        assert_deep_bf16(got, ref, 2, "two layers, full vocabulary")


def test_the_head_and_the_samplers_at_128256_columns():
    """The head product with its 1,002 weight tiles, and argmax and the temperature / top-p
    sampler over 128,256 scores, against float64 and the plain sampler."""
    from borrowed_compute_b200 import ops

    r = np.random.default_rng(4)
    E = CONFIG_8B["hidden_size"]
    w = torch.empty((VOCAB, E), dtype=torch.bfloat16, device="cuda")
    ops.random_normal(w, 12345, 0.02)
    x = torch.from_numpy(r.standard_normal((3, E)).astype(np.float32)).cuda().bfloat16()
    scores = torch.empty((3, VOCAB), dtype=torch.float32, device="cuda")
    ops.gemm_tc(x, w, scores, ops.EPI_STORE_F32)
    want = x.double() @ w.double().T
    assert float((scores.double() - want).abs().max()) <= 1e-3 * (1.0 + float(want.abs().max()))
    simt = torch.empty_like(scores)
    ops.gemm_simt(x, w, simt, ops.EPI_STORE_F32)
    assert float((simt.double() - want).abs().max()) <= 1e-3 * (1.0 + float(want.abs().max()))
    # samplers: the scores above, sharpened so that the nucleus is a few hundred tokens
    sharp = (scores * 4.0).contiguous()
    host = sharp.cpu().numpy()
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    ops.argmax(sharp, out)
    assert out.tolist() == [plain_llama.argmax(row) for row in host]
    tied = sharp.clone()
    tied[0, 100_000] = tied[0, 77] = float(tied[0].max()) + 1.0           # equal maxima far apart: the first wins
    ops.argmax(tied, out)
    assert out.tolist()[0] == 77
    # One draw a row with mixed settings.  Where the uniform draw lands within rounding of a
    # boundary between two tokens either may be picked; such rows must be rare and the token
    # picked must hold the draw within that margin.
    rows = sharp[[0, 1, 2, 0, 1, 2, 0, 1, 2, 0, 1, 2]].contiguous()
    settings = [(0.8, 0.9), (1.0, 1.0), (0.0, 1.0), (1.5, 0.5), (0.3, 0.95), (1.0, 0.99)] * 2
    temperature = torch.tensor([t for t, _ in settings], dtype=torch.float32, device="cuda")
    top_p = torch.tensor([p for _, p in settings], dtype=torch.float32, device="cuda")
    seeds = [0x9E3779B97F4A7C15 ^ i for i in range(12)]
    seed = torch.tensor([sd - (1 << 64) if sd >= (1 << 63) else sd for sd in seeds], dtype=torch.int64, device="cuda")
    steps = torch.tensor([0, 5, 2047, 2048, 9, 100, 7, 8191, 3, 64, 65, 1000], dtype=torch.int32, device="cuda")
    out = torch.empty(12, dtype=torch.int32, device="cuda")
    ops.sample(rows, temperature, top_p, seed, steps, out)
    got, same = out.tolist(), 0
    for i, (t, p) in enumerate(settings):
        row, step = host[i % 3], int(steps[i])
        want_id = plain_llama.sample(row, t, p, seeds[i], step)
        if got[i] == want_id:
            same += 1
            continue
        order, wts = plain_llama.nucleus(row, t, p)
        assert got[i] in order, f"row {i}: token {got[i]} is outside the nucleus"
        u = plain_llama.uniform((seeds[i] ^ ((step * 0x9E3779B97F4A7C15) & plain_llama.MASK64)) & plain_llama.MASK64) * wts.sum()
        cum = np.cumsum(wts)
        j = order.index(got[i])
        assert (cum[j - 1] if j else 0.0) - 1e-4 * wts.sum() <= u <= cum[j] + 1e-4 * wts.sum(), f"row {i}: token {got[i]} does not hold the draw"
    assert same >= 10


def test_prompt_attention_past_256_pages_of_one_sequence():
    """A sequence that continues at position 16,500 reads more pages than the tcgen05 prompt
    kernel keeps a list of in shared memory (256): the rows' scores over all 16,600 positions
    against float64, with one far key made to stand out."""
    from borrowed_compute_b200 import ops

    r = np.random.default_rng(6)
    H, G, D, start, new = 2, 1, 64, 16500, 100
    total = start + new
    pages = -(-total // 64)
    k = r.standard_normal((total, G, D)).astype(np.float32) * 0.5
    v = r.standard_normal((total, G, D)).astype(np.float32)
    q = r.standard_normal((new, H, D)).astype(np.float32) * 0.5
    k[300] = q[7, 1] * 6.0                       # row 7's second head finds position 300, in the fifth page, among sixteen thousand
    order = r.permutation(pages + 3)[:pages]     # the sequence's pages lie scattered in the pool
    kc = torch.zeros((pages + 3, G, 64, D), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    kb, vb = torch.from_numpy(k).bfloat16(), torch.from_numpy(v).bfloat16()
    for i, p in enumerate(order):
        n = min(64, total - 64 * i)
        kc[p, :, :n] = kb[64 * i:64 * i + n].permute(1, 0, 2).cuda()
        vc[p, :, :n] = vb[64 * i:64 * i + n].permute(1, 0, 2).cuda()
    table = torch.full((1, pages + 8), -1, dtype=torch.int32)
    table[0, :pages] = torch.from_numpy(order.astype(np.int32))
    qkv = torch.zeros((new, (H + 2 * G) * D), dtype=torch.bfloat16, device="cuda")
    qb = torch.from_numpy(q).bfloat16()
    qkv[:, :H * D] = qb.reshape(new, H * D).cuda()
    out = torch.empty((new, H * D), dtype=torch.bfloat16, device="cuda")
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    assert ops.attention_prefill_tc_accepts(H, G, D, qkv, (H + 2 * G) * D)
    ops.attention_prefill(qkv, (H + 2 * G) * D, kc, vc, table.cuda(), i32([0, new]), i32([0]), i32([start]), out, 1, new, H, G, D, use_tc=True)
    torch.cuda.synchronize()
    assert ops.attention_prefill_tc_status() == 0
    k64, v64, q64 = kb.double().numpy(), vb.double().numpy(), qb.double().numpy()
    ref = np.zeros((new, H, D))
    for i in range(new):
        for h in range(H):
            s = k64[: start + i + 1, 0] @ q64[i, h] / 8.0
            p = np.exp(s - s.max())
            ref[i, h] = (p / p.sum()) @ v64[: start + i + 1, 0]
            if (i, h) == (7, 1):
                assert p[300] / p.sum() > 0.5, "the far key dominates its row"
    got = out.float().cpu().numpy().astype(np.float64).reshape(new, H, D)
    assert np.abs(got - ref).max() <= 2.0 ** -6 * (1 + np.abs(ref).max())
