"""The generation loop's decisions, driven through a backend that needs no device."""

from __future__ import annotations

import pytest

from borrowed_compute_b200.engine.batch import StepEntry, plan_step
from borrowed_compute_b200.engine.generate import Backend, run_generation
from borrowed_compute_b200.sampling import Sampling


class Scripted(Backend):
    """Every sequence's next token is (last token + 1) mod 50; records what the loop asks."""

    def __init__(self, max_batch, context=0):
        self.max_batch, self.context = max_batch, context
        self.live, self.log = set(), []

    def start(self, indices, prompts, samplings):
        assert not self.live, "a new batch started before the last one ended"
        assert len(indices) <= self.max_batch
        self.live |= set(indices)
        self.log.append(("start", tuple(indices), tuple(len(p) for p in prompts)))
        return [(p[-1] + 1) % 50 for p in prompts]

    def advance(self, indices, tokens):
        assert set(indices) <= self.live
        self.log.append(("advance", tuple(indices)))
        return [(t + 1) % 50 for t in tokens]

    def finish(self, index):
        assert index in self.live, "a sequence was finished twice"
        self.live.remove(index)
        self.log.append(("finish", index))


def test_counts_tokens_and_frees_everything():
    b = Scripted(max_batch=4)
    out, stats = run_generation(b, [[1], [10, 11], [20, 21, 22]], 5, [Sampling()] * 3)
    assert out == [[2, 3, 4, 5, 6], [12, 13, 14, 15, 16], [23, 24, 25, 26, 27]]
    assert not b.live and stats.generated == 15 and stats.prompt_tokens == 6 and stats.passes == 4 and stats.first_tokens == 3
    assert [e for e in b.log if e[0] == "advance"] == [("advance", (0, 1, 2))] * 4


def test_stop_ids_end_a_sequence_and_are_not_emitted():
    b = Scripted(max_batch=4)
    out, stats = run_generation(b, [[1], [10], [30]], 8, [Sampling()] * 3, stop_ids=[13, 31])
    assert out == [[2, 3, 4, 5, 6, 7, 8, 9], [11, 12], []]
    advances = [e[1] for e in b.log if e[0] == "advance"]
    assert advances[0] == (0, 1) and advances[1] == (0, 1) and advances[2] == (0,)   # shorter requests leave early
    assert b.log.index(("finish", 2)) < b.log.index(("advance", (0, 1)))
    assert not b.live


def test_batches_follow_one_another():
    b = Scripted(max_batch=2)
    prompts = [[i] for i in range(5)]
    seen = []
    out, stats = run_generation(b, prompts, 3, [Sampling()] * 5, on_token=lambda i, t: seen.append((i, t)))
    assert out == [[i + 1, i + 2, i + 3] for i in range(5)]
    assert [e[1] for e in b.log if e[0] == "start"] == [(0, 1), (2, 3), (4,)]
    assert sorted(seen) == sorted((i, t) for i, o in enumerate(out) for t in o)
    assert stats.passes == 6 and stats.first_tokens == 5


def test_limits_are_checked_first():
    b = Scripted(max_batch=2, context=10)
    with pytest.raises(ValueError, match="empty"):
        run_generation(b, [[1], []], 3, [Sampling()] * 2)
    with pytest.raises(ValueError, match="exceed the context"):
        run_generation(b, [[1] * 8], 3, [Sampling()])
    with pytest.raises(ValueError, match="one Sampling"):
        run_generation(b, [[1]], 3, [])
    assert b.log == []
    out, _ = run_generation(b, [[1] * 7], 3, [Sampling()])
    assert len(out[0]) == 3
    out, stats = run_generation(Scripted(2), [[1]], 0, [Sampling()])
    assert out == [[]] and stats.passes == 0


def test_sampling_parameters():
    assert Sampling().greedy and not Sampling(temperature=0.7).greedy
    assert Sampling(seed=(1 << 64) - 1).seed_as_int64 == -1 and Sampling(seed=5).seed_as_int64 == 5
    with pytest.raises(ValueError):
        Sampling(top_p=0.0)
    with pytest.raises(ValueError):
        Sampling(seed=-1)


def test_plan_step_flattens_and_pads():
    plan = plan_step([StepEntry(3, [7, 8, 9], want=(0, 2)), StepEntry(1, [5], want=(0,))], starts=[10, 0], pad_rows_to=8)
    assert plan.rows == 4 and plan.padded_rows == 8 and plan.seqs == 2 and not plan.decode
    assert list(plan.tokens) == [7, 8, 9, 5, 0, 0, 0, 0]
    assert list(plan.row_pos) == [10, 11, 12, 0, 0, 0, 0, 0]
    assert list(plan.row_slot) == [3, 3, 3, 1, -1, -1, -1, -1]
    assert list(plan.seq_rows) == [0, 3, 4] and list(plan.want_rows) == [0, 2, 3]
    assert plan.max_new == 3 and plan.max_total == 13
    assert sum(n for _, n in plan.layout()) == plan.packed().size
    assert plan_step([StepEntry(0, [1]), StepEntry(2, [3])], [4, 9]).decode
    with pytest.raises(ValueError, match="twice"):
        plan_step([StepEntry(0, [1]), StepEntry(0, [3])], [0, 0])
    with pytest.raises(ValueError, match="at least one token"):
        plan_step([StepEntry(0, [])], [0])
    with pytest.raises(ValueError, match="outside"):
        plan_step([StepEntry(0, [1, 2], want=(2,))], [0])


class Chaining(Scripted):
    """The same script, but a pass can be begun before the last one's ids are read: it is
    then fed the ids the backend itself holds, as an engine feeds them on the device."""

    def __init__(self, max_batch, context=0, refuse_every=0):
        super().__init__(max_batch, context)
        self.held, self.last, self.unread, self.refuse_every, self.asked = {}, None, 0, refuse_every, 0

    def start(self, indices, prompts, samplings):
        first = super().start(indices, prompts, samplings)
        self.last = None
        return first

    def begin(self, indices, tokens):
        from borrowed_compute_b200.engine.generate import Pending

        assert set(indices) <= self.live
        if tokens is None:
            self.asked += 1
            if self.last != tuple(indices) or (self.refuse_every and self.asked % self.refuse_every == 0):
                return None                                  # cannot follow on: the loop must read the ids first
            tokens = [self.held[i] for i in indices]
            self.log.append(("chained", tuple(indices)))
        else:
            assert self.unread == 0, "a pass fed by the host while ids of an earlier one are unread"
            self.log.append(("advance", tuple(indices)))
        ids = [(t + 1) % 50 for t in tokens]
        self.held.update(zip(indices, ids))
        self.last = tuple(indices)
        self.unread += 1
        assert self.unread <= 2, "more than one pass ahead of the host"
        owner = self

        class Later(Pending):
            def ids(self):
                owner.unread -= 1
                return ids

        return Later()

    def finish(self, index):
        super().finish(index)
        self.last = None


@pytest.mark.parametrize("refuse_every", [0, 3])
def test_passes_begun_ahead_give_the_same_tokens(refuse_every):
    import random

    rnd = random.Random(4)
    for trial in range(40):
        n = rnd.randint(1, 7)
        prompts = [[rnd.randrange(50) for _ in range(rnd.randint(1, 4))] for _ in range(n)]
        max_tokens = rnd.randint(0, 9)
        stops = [rnd.randrange(50) for _ in range(rnd.randint(0, 6))]
        plain = Scripted(max_batch=3)
        want, want_stats = run_generation(plain, prompts, max_tokens, [Sampling()] * n, stop_ids=stops)
        ahead = Chaining(max_batch=3, refuse_every=refuse_every)
        got, stats = run_generation(ahead, prompts, max_tokens, [Sampling()] * n, stop_ids=stops)
        assert got == want and not ahead.live and ahead.unread == 0
        assert stats.generated == want_stats.generated and stats.passes >= want_stats.passes
        assert sorted(e[1] for e in ahead.log if e[0] == "finish") == list(range(n)), "every sequence is finished exactly once"


def test_a_pass_begun_ahead_is_never_a_sequences_last_by_count():
    b = Chaining(max_batch=2)
    out, stats = run_generation(b, [[1], [10]], 4, [Sampling()] * 2)
    assert out == [[2, 3, 4, 5], [11, 12, 13, 14]]
    # token 1 comes from the prompts; tokens 2, 3 and 4 from three passes, the last of which is not run ahead of
    assert [e[0] for e in b.log if e[0] in ("advance", "chained")] == ["advance", "chained", "chained"]
    assert stats.passes == 3
    # a stop id is seen one pass late: the sequence's row of the pass in flight runs for nothing, then it leaves
    b = Chaining(max_batch=2)
    out, stats = run_generation(b, [[1], [10]], 9, [Sampling()] * 2, stop_ids=[13])
    assert out == [[2, 3, 4, 5, 6, 7, 8, 9, 10], [11, 12]]
    steps = [e for e in b.log if e[0] in ("advance", "chained", "finish")]
    assert steps[:4] == [("advance", (0, 1)), ("chained", (0, 1)), ("chained", (0, 1)), ("finish", 1)]
    assert steps[4] == ("advance", (0,)) and not b.live


def test_a_stop_id_can_be_kept_as_the_last_id():
    for backend in (Scripted(max_batch=4), Chaining(max_batch=4)):
        seen = []
        out, stats = run_generation(backend, [[1], [10], [30]], 8, [Sampling()] * 3, stop_ids=[13, 31], include_stop=True,
                                    on_token=lambda i, t: seen.append((i, t)))
        assert out == [[2, 3, 4, 5, 6, 7, 8, 9], [11, 12, 13], [31]] and not backend.live
        assert stats.generated == 12 and sorted(seen) == sorted((i, t) for i, o in enumerate(out) for t in o)
    out, _ = run_generation(Scripted(max_batch=1), [[10]], 2, [Sampling()], stop_ids=[13], include_stop=True)
    assert out == [[11, 12]], "the count ends a sequence before a stop id that lies past it"
