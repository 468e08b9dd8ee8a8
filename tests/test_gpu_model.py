"""The engine against the plain implementation: whole prompts, the last 32 tokens one by one,
batches of unequal lengths with slot reuse, long decoding, first tokens, padding; in float32
and in bfloat16, for both tiny configurations."""

from __future__ import annotations

import numpy as np
import pytest

import plain_llama
from conftest import TINY, seeded_tokens, tolerance

pytestmark = pytest.mark.gpu

CASES = [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")]


@pytest.fixture(scope="module")
def engines(model_folders):
    from borrowed_compute_b200.engine import Engine

    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            folder, cfg, weights = model_folders(name, dtype)
            made[(name, dtype)] = (Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=6), cfg, weights)
        return made[(name, dtype)]

    return get


_plain_cache = {}


def plain(name, dtype, cfg, weights, tokens):
    key = (name, dtype, tuple(tokens))
    if key not in _plain_cache:
        _plain_cache[key] = plain_llama.logits(cfg, weights, tokens)
    return _plain_cache[key]


def requests_for(name):
    cfg = TINY[name]
    lengths = {"A": [5, 17, 1, 40, 100], "B": [1, 9, 33, 70, 150]}[name]
    return [seeded_tokens(100 + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)]


def close(got, ref, dtype, what):
    tol = tolerance(dtype, ref)
    err = float(np.abs(got - ref).max())
    assert err <= tol, f"{what}: max error {err:.3e} over tolerance {tol:.3e}"


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(engines, name, dtype):
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, weights = engines(name, dtype)
    for tokens in requests_for(name):
        slot = eng.acquire()
        got = eng.step([StepEntry(slot, tokens, want=tuple(range(len(tokens))))]).cpu().numpy()
        eng.release(slot)
        close(got, plain(name, dtype, cfg, weights, tokens), dtype, f"whole prompt of {len(tokens)}")
    eng.cache.slots.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(engines, name, dtype):
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, weights = engines(name, dtype)
    for tokens in requests_for(name):
        if len(tokens) <= 32:
            continue
        ref = plain(name, dtype, cfg, weights, tokens)
        cut = len(tokens) - 32
        slot = eng.acquire()
        rows = [eng.step([StepEntry(slot, tokens[:cut], want=tuple(range(cut)))]).cpu().numpy()]
        for t in tokens[cut:]:
            rows.append(eng.step([StepEntry(slot, [t], want=(0,))]).cpu().numpy())
        eng.release(slot)
        got = np.concatenate(rows)
        # The first decoded token and the prompt's end are where a cache fault would show first.
        close(got[cut - 1:cut + 1], ref[cut - 1:cut + 1], dtype, "prompt end and first decoded token")
        close(got, ref, dtype, f"prompt of {cut} then 32 single tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_one_after_another(engines, name, dtype):
    """Two batches through the same slots; within a batch all prompts run in one step, then
    one token each, and shorter requests end (and free their slot) earlier."""
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, weights = engines(name, dtype)
    reqs = requests_for(name)
    vocab = cfg["vocab_size"]
    batches = [[reqs[0], reqs[1], reqs[2]], [reqs[3], reqs[1][::-1], reqs[0][::-1], reqs[2]]]
    for b, batch in enumerate(batches):
        # Each request: a prompt part fed at once, then its remaining tokens one a step.
        decode_n = [min(len(r) - 1, 3 + 2 * i) for i, r in enumerate(batch)]
        prompts = [r[: len(r) - d] for r, d in zip(batch, decode_n)]
        slots = [eng.acquire() for _ in batch]
        got = [[] for _ in batch]
        scores = eng.step([StepEntry(s, p, want=tuple(range(len(p)))) for s, p in zip(slots, prompts)]).cpu().numpy()
        at = 0
        for i, p in enumerate(prompts):
            got[i].append(scores[at:at + len(p)])
            at += len(p)
        live = [i for i in range(len(batch)) if decode_n[i] > 0]
        for i in range(len(batch)):
            if decode_n[i] == 0:
                eng.release(slots[i])
        step = 0
        while live:
            entries = [StepEntry(slots[i], [batch[i][len(prompts[i]) + step]], want=(0,)) for i in live]
            scores = eng.step(entries).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(scores[j:j + 1])
            step += 1
            for i in list(live):
                if step >= decode_n[i]:
                    eng.release(slots[i])
                    live.remove(i)
        eng.cache.slots.check()
        for i, r in enumerate(batch):
            close(np.concatenate(got[i]), plain(name, dtype, cfg, weights, r), dtype, f"batch {b} request {i} (length {len(r)})")
    assert eng.cache.slots.live() == []
    assert vocab == scores.shape[1]


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding_crosses_pages(engines, name, dtype):
    """One token a step from the first position on, past two page boundaries (64, 128 for
    B; 64 for A) and past the scaled rotary range of B."""
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, weights = engines(name, dtype)
    n = {"A": 100, "B": 150}[name]
    tokens = seeded_tokens(7, n, cfg["vocab_size"])
    ref = plain(name, dtype, cfg, weights, tokens)
    slot = eng.acquire()
    got = np.concatenate([eng.step([StepEntry(slot, [t], want=(0,))]).cpu().numpy() for t in tokens])
    eng.release(slot)
    close(got[:4], ref[:4], dtype, "the first tokens of a sequence")
    close(got, ref, dtype, f"{n} tokens decoded one by one")


@pytest.mark.parametrize("name,dtype", CASES)
def test_padding_rows_change_nothing(engines, name, dtype):
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, weights = engines(name, dtype)
    reqs = requests_for(name)[:3]
    out = []
    for pad in (1, 16):
        slots = [eng.acquire() for _ in reqs]
        out.append(eng.step([StepEntry(s, r, want=(len(r) - 1,)) for s, r in zip(slots, reqs)], pad_rows_to=pad).cpu().numpy())
        for s in slots:
            eng.release(s)
    assert np.array_equal(out[0], out[1]), "padding rows changed a result"


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_cuts_agree_to_the_bit(engines, name):
    """In float32 every row's sums run in an order that depends on the row alone, so a
    prompt cut into steps, or batched with others, gives the same bits."""
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, _ = engines(name, "float32")
    a, b = requests_for(name)[3], requests_for(name)[1]
    s = eng.acquire()
    whole = eng.step([StepEntry(s, a, want=tuple(range(len(a))))]).cpu().numpy()
    eng.release(s)
    s, s2 = eng.acquire(), eng.acquire()
    first = eng.step([StepEntry(s2, b, want=()), StepEntry(s, a[:7], want=tuple(range(7)))]).cpu().numpy()
    rest = [eng.step([StepEntry(s, [t], want=(0,)), StepEntry(s2, [1], want=())]).cpu().numpy() for t in a[7:]]
    eng.release(s)
    eng.release(s2)
    assert np.array_equal(np.concatenate([first] + rest), whole)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_decode_steps_staged_ahead_and_every_way_out_of_them(engines, name, dtype):
    """After a decode step the engine stages the next one for the same sequences.  The
    staged step is used when exactly they come again, and dropped when they come in another
    order, when one of them has ended and its slot is taken by a new sequence, or after a
    cut back; the scores match the plain implementation every time."""
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, weights = engines(name, dtype)
    assert eng.use_graphs
    V = cfg["vocab_size"]
    seqs = [seeded_tokens(300 + i, n, V) for i, n in enumerate([70, 9, 63, 30])]
    held = [3, 2, 3, 5]          # tokens of each sequence that its prompt step takes
    slots = [eng.acquire() for _ in seqs]
    eng.step([StepEntry(s, t[:h], want=()) for s, t, h in zip(slots, seqs, held)])
    at = list(held)

    def decode(order):
        scores = eng.step([StepEntry(slots[i], (seqs[i][at[i]],), want=(0,)) for i in order]).float().cpu().numpy()
        for row, i in zip(scores, order):
            close(row, plain(name, dtype, cfg, weights, seqs[i][:at[i] + 1])[-1], dtype, f"sequence {i} position {at[i]}")
            at[i] += 1

    decode([0, 1, 2, 3])
    assert eng._ahead is not None
    decode([0, 1, 2, 3])                  # the staged step
    decode([0, 1, 2, 3])
    decode([3, 2, 1, 0])                  # another order: not the staged step
    decode([3, 2, 1, 0])
    decode([0, 2])                        # fewer sequences
    decode([0, 2])
    eng.release(slots[1])                 # a sequence ends, a new one takes its slot
    seqs[1] = seeded_tokens(400, 40, V)
    slots[1] = eng.acquire()
    eng.step([StepEntry(slots[1], seqs[1][:4], want=())])
    at[1] = 4
    decode([0, 1, 2, 3])
    decode([0, 1, 2, 3])
    eng.rollback(slots[3], at[3] - 2)     # a cut back between two steps of the same sequences
    at[3] -= 2
    assert eng._ahead is None
    decode([0, 1, 2, 3])
    for _ in range(6):                    # sequence 2 crosses a page edge on staged steps
        decode([0, 1, 2, 3])
    for s in slots:
        eng.release(s)
    eng.cache.slots.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_going_back_reproduces(engines, dtype):
    """Re-running a position after cutting the cache back gives the same scores again
    (crates/bc-infer/src/model.rs:532-534)."""
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, _ = engines("B", dtype)
    tokens = requests_for("B")[3]
    s = eng.acquire()
    eng.step([StepEntry(s, tokens[:60], want=())])
    first = eng.step([StepEntry(s, tokens[60:], want=tuple(range(10)))]).cpu().numpy()
    eng.rollback(s, 60)
    again = eng.step([StepEntry(s, tokens[60:], want=tuple(range(10)))]).cpu().numpy()
    eng.release(s)
    assert np.array_equal(first, again)


def test_guards(engines):
    from borrowed_compute_b200.config import CacheError
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, _ = engines("A", "float32")
    s = eng.acquire()
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.step([StepEntry(s, [cfg["vocab_size"]], want=(0,))])
    with pytest.raises(CacheError):
        eng.step([StepEntry(s, [1] * (eng.max_seq + 1), want=())])
    with pytest.raises(ValueError):
        eng.step([StepEntry(s, [], want=())])
    eng.release(s)
    with pytest.raises(CacheError):
        eng.step([StepEntry(s, [1], want=(0,))])
    with pytest.raises(CacheError):
        eng.release(s)
