"""The generation loop's decisions, with a fake engine (no GPU)."""

import pytest
import torch

from reflex_b200 import ContextOverflow, InvalidInput, SamplingParams
from reflex_b200.cache import Cache, KVSpec
from reflex_b200.engine.generate import GenerationStats, generate, plan_batches
from reflex_b200.sampling.params import uniform


class FakeEngine:
    """Next token = (last token + 1) % vocab; keeps the real cache bookkeeping."""

    def __init__(self, max_tokens=1024, max_positions=512, vocab=50, max_slots=None):
        self.cache = Cache({0: KVSpec(1, 16)}, max_tokens, max_positions, torch.float32, None,
                           max_slots=max_slots)
        self.vocab = vocab
        self.steps = []
        self.slot_history = []

    def open(self):
        s = self.cache.take_slot()
        self.slot_history.append(s)
        return s

    def close(self, s):
        self.cache.give_slot(s)

    def step(self, entries):
        growth = [(s, len(t)) for s, t, _ in entries]
        self.cache.reserve(growth)
        self.cache.commit(growth)
        self.steps.append([(s, list(t)) for s, t, _ in entries])
        rows = []
        for s, toks, want in entries:
            for w in want:
                row = torch.zeros(self.vocab)
                row[(toks[w] + 1) % self.vocab] = 1.0
                rows.append(row)
        return torch.stack(rows)


def greedy(logits, requests, steps):
    return logits.argmax(dim=1).tolist()


def test_counts_and_feedback():
    e = FakeEngine()
    out = generate(e, [[3, 4, 5], [10]], 4, greedy)
    assert out == [[6, 7, 8, 9], [11, 12, 13, 14]]
    assert [len(s) for s in e.steps] == [2, 2, 2, 2]  # one prefill + 3 decode steps
    assert e.steps[0][0][1] == [3, 4, 5] and e.steps[1][0][1] == [6]
    assert e.cache.slots.held_count == 0


def test_stop_token_is_kept_and_ends_only_its_request():
    e = FakeEngine()
    stats = GenerationStats()
    out = generate(e, [[1], [20], [30]], 10, greedy, stop_token_ids=[3, 21], stats=stats)
    assert out[0] == [2, 3]
    assert out[1] == [21]  # a stop token as the first token: exactly one token
    assert out[2] == list(range(31, 41))
    assert [len(s) for s in e.steps] == [3, 2] + [1] * 8
    assert stats.prefill_tokens == 3 and stats.decode_steps == 9 and stats.decode_tokens == 2 + 8
    assert e.cache.slots.held_count == 0
    assert all(g.pool.held_count == 0 for g in e.cache.kv_groups)


def test_max_new_tokens_and_input_checks():
    e = FakeEngine()
    with pytest.raises(InvalidInput) as err:
        generate(e, [[1]], 0, greedy)
    assert "max_new_tokens must be at least 1" in str(err.value)
    with pytest.raises(InvalidInput):
        generate(e, [[1], []], 3, greedy)
    with pytest.raises(InvalidInput):
        generate(e, [], 3, greedy)
    with pytest.raises(ContextOverflow):
        generate(e, [[1] * 510], 3, greedy)
    assert generate(e, [[1] * 509], 3, greedy) == [[2, 3, 4]]


def test_batches_one_after_another_reuse_slots():
    e = FakeEngine(max_tokens=64 * 3, max_slots=3)
    prompts = [[i] for i in range(7)]
    stats = GenerationStats()
    out = generate(e, prompts, 2, greedy, stats=stats)
    assert out == [[i + 1, i + 2] for i in range(7)]
    assert stats.batches == 3
    assert set(e.slot_history) == {0, 1, 2} and len(e.slot_history) == 7
    assert e.cache.slots.held_count == 0


def test_plan_batches():
    assert plan_batches([10, 10, 10], 5, 64 * 2, 8) == [[0, 1], [2]]
    assert plan_batches([10] * 5, 5, 64 * 100, 2) == [[0, 1], [2, 3], [4]]
    assert plan_batches([100, 10], 30, 64 * 3, 8) == [[0], [1]]  # 130 -> 3 pages
    with pytest.raises(ContextOverflow):
        plan_batches([200], 5, 128, 8)


def test_slots_are_given_back_when_a_step_fails():
    e = FakeEngine()

    def boom(logits, requests, steps):
        raise RuntimeError("picker failed")

    with pytest.raises(RuntimeError):
        generate(e, [[1], [2]], 3, boom)
    assert e.cache.slots.held_count == 0


def test_on_token_sees_every_token_in_order():
    e = FakeEngine()
    seen = []
    generate(e, [[1], [7]], 3, greedy, on_token=lambda i, t: seen.append((i, t)))
    assert seen == [(0, 2), (1, 8), (0, 3), (1, 9), (0, 4), (1, 10)]


def test_sampling_params_meanings():
    assert SamplingParams().is_greedy()
    assert SamplingParams(temperature=float("nan")).is_greedy()
    assert SamplingParams(temperature=-1.0).is_greedy()
    assert not SamplingParams(temperature=0.7).is_greedy()
    SamplingParams(temperature=0.0, top_k=0).validate()  # ignored when greedy
    for bad in (dict(temperature=float("inf")), dict(temperature=1.0, top_k=0),
                dict(temperature=1.0, top_p=1.5), dict(temperature=1.0, top_p=float("nan"))):
        with pytest.raises(InvalidInput):
            SamplingParams(**bad).validate()


def test_uniform_depends_only_on_seed_request_step():
    a = [uniform(1, r, s) for r in range(4) for s in range(50)]
    assert a == [uniform(1, r, s) for r in range(4) for s in range(50)]
    assert all(0.0 <= u < 1.0 for u in a)
    assert len(set(a)) > 190
    assert abs(sum(a) / len(a) - 0.5) < 0.08
    assert uniform(2, 0, 0) != uniform(1, 0, 0)


# ---- the loop that keeps the device one step ahead of the host ---------------


class AheadEngine(FakeEngine):
    """Adds `step_decode`, and checks what the ahead loop must respect: a slot
    is never given back while a step that carries its row is still 'running'
    (here: until the pick made from that step's logits has been waited for)."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.in_flight = []  # slots of steps whose picks have not been waited for

    def step(self, entries):
        self.in_flight.append([s for s, _, _ in entries])
        return super().step(entries)

    def step_decode(self, seqs, tokens_dev):
        toks = [int(t) for t in tokens_dev]
        assert len(toks) == len(seqs)
        return self.step([(s, [t], [0]) for s, t in zip(seqs, toks)])

    def close(self, s):
        assert all(s not in slots for slots in self.in_flight), "slot freed under a running step"
        super().close(s)


class FakePending:
    def __init__(self, engine, ids):
        self.engine, self.dev, self.ids = engine, torch.tensor(ids, dtype=torch.int32), ids

    def wait(self):
        self.engine.in_flight.pop(0)  # picks are waited for in order: the oldest step is over
        return list(self.ids)


def ahead_pick(engine):
    return lambda logits, requests, steps: FakePending(engine, logits.argmax(dim=1).tolist())


@pytest.mark.parametrize("prompts,n,stops", [
    ([[3, 4, 5], [10]], 4, []),
    ([[1], [20], [30]], 10, [3, 21]),
    ([[1], [20], [30]], 1, []),
    ([[5], [6], [7], [8], [9]], 6, [8, 9, 12]),
    ([[40], [41]], 7, [44, 45]),  # both end on the same step by stop tokens
])
def test_the_ahead_loop_returns_the_same_tokens_and_frees_everything(prompts, n, stops):
    plain = FakeEngine(max_slots=3)
    want_stats = GenerationStats()
    want = generate(plain, prompts, n, greedy, stop_token_ids=stops, max_batch=3, stats=want_stats)
    e = AheadEngine(max_slots=3)
    stats = GenerationStats()
    seen = []
    got = generate(e, prompts, n, greedy, stop_token_ids=stops, max_batch=3, stats=stats,
                   pick_async=ahead_pick(e), on_token=lambda i, t: seen.append((i, t)))
    assert got == want
    assert sorted(seen) == sorted((i, t) for i, out in enumerate(want) for t in out)
    assert e.cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in e.cache.kv_groups)
    assert not e.in_flight
    assert (stats.prefill_tokens, stats.decode_tokens, stats.batches) == \
        (want_stats.prefill_tokens, want_stats.decode_tokens, want_stats.batches)
    assert stats.decode_steps == want_stats.decode_steps
    # a request that picked a stop token rides along for at most one more step
    assert sum(len(st) for st in plain.steps) <= sum(len(st) for st in e.steps) \
        <= sum(len(st) for st in plain.steps) + len(prompts)


def test_slots_taken_before_an_open_fails_are_given_back():
    """If taking a slot fails part-way through a batch's start, the slots
    already taken go back: nothing stays held for the life of the engine."""
    from reflex_b200 import OutOfMemory

    class Stingy(FakeEngine):
        def open(self):
            if self.cache.slots.held_count >= 2:
                raise OutOfMemory("no slot left (made up by the test)")
            return super().open()

    e = Stingy()
    with pytest.raises(OutOfMemory):
        generate(e, [[1], [2], [3]], 2, greedy)
    assert e.cache.slots.held_count == 0
